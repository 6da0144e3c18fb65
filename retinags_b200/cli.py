"""Process set-up and dispatch for ``main.py`` (see there for the command line)."""
from __future__ import annotations

import datetime
import logging
import os
import time
import traceback

import torch
import torch.distributed as dist

from .config import build_parser
from .utils.general import seed_everything


def setup_distributed(device_kind: str):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and device_kind != "cpu"
    if use_cuda:
        torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = dict(device_id=torch.device("cuda", local)) if use_cuda else {}
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=6000), **kw)
    return rank, world, local


def main(argv=None) -> int:
    parser, lp, op, pp = build_parser()
    args = parser.parse_args(argv)
    # --detect_anomaly: the step engine checks loss sums and gradients for non-finite values after every backward
    # (retinags_b200/engine.py); no autograd graph exists on the training path
    seed_everything(0)
    rank, world, _ = setup_distributed(args.device)
    if world > 2 ** args.bvh_depth:
        raise SystemExit(f"WORLD_SIZE {world} needs bvh_depth >= {max(world - 1, 0).bit_length()}")
    os.makedirs("debugger", exist_ok=True)
    dbg = logging.getLogger("debugger")
    dbg.addHandler(logging.FileHandler(f"debugger/debug_{rank}_{time.strftime('%Y_%m_%d_%H')}.txt", mode="a"))
    dbg.setLevel(logging.INFO)
    code = 0
    trainer = None
    try:
        from .trainer import Trainer
        scene = None
        if args.synthetic:
            from .data.synthetic_scene import build_synthetic_scene
            scene = build_synthetic_scene(args.synthetic, lp.extract(args))
        trainer = Trainer(args, lp.extract(args), op.extract(args), pp.extract(args), scene=scene)
        if args.EVAL_ONLY:
            trainer.eval()
        else:
            trainer.train()
        if rank == 0 and not args.quiet:
            print("\nTraining complete." if not args.EVAL_ONLY else "\nEvaluation complete.")
    except Exception as exc:
        dbg.error(traceback.format_exc())
        traceback.print_exc()
        if trainer is not None and getattr(trainer, "watchdog", None) is not None:
            trainer.watchdog.report_failure(repr(exc))  # peers stop at their next step instead of hanging
        code = 1
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass
    return code
