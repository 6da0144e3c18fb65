#!/usr/bin/env python
"""Headline benchmark: training views/s at 62.9M Gaussians, 1600x1036, on N B200s of one node.

Own arm (default): the framework's trainer on a seeded synthetic cluster scene (random-init
Gaussians, SH degree 3, fp32), 2^k sub-models for N = 2^k GPUs (strong scaling: the scene is fixed),
two views per step.  Reference arm (``--impl reference``): the unmodified reference installed
under ``baseline/_ref`` run through its own trainer on the same synthetic scene written to disk.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--gaussians", type=int, default=62_900_000)
    ap.add_argument("--width", type=int, default=1600)
    ap.add_argument("--height", type=int, default=1036)
    ap.add_argument("--batch", type=int, default=2, help="views per step (MAX_BATCH_SIZE of the 8-GPU config)")
    ap.add_argument("--gt-gaussians", type=int, default=6_000_000)
    ap.add_argument("--transport", default="auto", choices=["auto", "peer", "nccl"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--borrow-refresh", type=int, default=8,
                    help="steps between recomputations of the border-Gaussian selection (the rows are re-sent every step)")
    ap.add_argument("--bvh-depth", type=int, default=None,
                    help="2^depth sub-models (default: one per GPU); more sub-models than GPUs are spread round-robin")
    ap.add_argument("--slabs", type=int, default=None, metavar="N",
                    help="two-slab forward with the nearest N/256 of the splats in the first slab (same as RGS_SLABS=1 "
                         "RGS_SLAB_FRACTION=N; default 6); 0 renders in one pass")
    ap.add_argument("--occlusion", type=int, default=None, choices=[0, 1],
                    help="occlusion culling between sub-models (finished-tile maps exchanged once per step)")
    ap.add_argument("--mode", default="train", choices=["train", "eval", "train-psnr", "trainer", "push", "city"],
                    help="train: the headline (training views/s of the step engine on an in-memory scene). The other modes "
                         "run the public trainer of either arm on one scene on disk (PNG targets, the initial model as a "
                         "PLY file): eval = eval render of --eval-frames test views (ms/frame, PSNR/SSIM/L1); train-psnr = "
                         "--epochs epochs over --train-views views, then that eval; trainer = views/s of Trainer.train(), "
                         "image decoding included (own arm only); push = the blend kernel with and without its fused "
                         "stores into the peers' compositing slots, against the NVLink roofline (own arm, >= 2 GPUs); "
                         "city = train steps on --scene, then one densification and one repartition with migration "
                         "(time, Gaussians moved, peak memory per rank)")
    ap.add_argument("--scene", default="cluster", choices=["cluster", "aerial"],
                    help="synthetic scene: the 64-cluster mixture of the headline, or the aerial city scene (ground plane "
                         "2000 x 2000 units + building-like vertical clusters, downward-tilted grid cameras)")
    ap.add_argument("--train-views", type=int, default=40)
    ap.add_argument("--eval-frames", type=int, default=20)
    ap.add_argument("--epochs", type=int, default=8)
    ap.add_argument("--pool-views", type=int, default=0,
                    help="form the batches from a seeded shuffle of this many training cameras (160 in the named config) "
                         "instead of consecutive cameras of a short list")
    ap.add_argument("--balance-batches", action="store_true",
                    help="with --pool-views: pair cameras whose estimated per-rank loads complement each other (the "
                         "trainer's --BALANCE_BATCHES)")
    ap.add_argument("--no-spatial-sort", action="store_true", help="keep the Gaussians in generation order (default: rows "
                    "are sorted along a Morton curve, the trainer's default as well)")
    ap.add_argument("--densify-threshold", type=float, default=2e-4, help="--mode city: screen-gradient threshold")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--phases", action="store_true", help="also time the phases of a step (extra loop, after the timed one)")
    ap.add_argument("--task-times", default="", help="with --phases: write the per-(camera, sub-model) render times of every "
                    "rank to <path>.rank<r>.json")
    ap.add_argument("--trace", default="", help="with --phases: write a Chrome trace of the phase loop to <path>.rank<r>.json")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    # nvidia-smi stalls the GPU for ~0.1 s while it attaches, so the sampler is started before the warm-up
    # steps and only the samples taken between mark_begin() and stop() are used.

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[tuple[float, str]] = []
        self.t_begin = 0.0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark_begin(self):
        self.t_begin = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for stamp, ln in self.lines:
            if stamp < self.t_begin:
                continue
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def run_own(args):
    import torch
    import torch.distributed as dist

    from retinags_b200.bench_session import BenchSession

    if args.slabs is not None:
        os.environ["RGS_SLABS"], os.environ["RGS_SLAB_FRACTION"] = ("1", str(args.slabs)) if args.slabs > 0 else ("0", "6")
    if args.occlusion is not None:
        os.environ["RGS_OCCLUSION"] = str(args.occlusion)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    sess = BenchSession(device=device, rank=rank, world=world, n_gaussians=args.gaussians, width=args.width,
                        height=args.height, batch=args.batch, n_views=(args.steps + args.warmup) * args.batch,
                        gt_gaussians=args.gt_gaussians, transport=args.transport, seed=args.seed,
                        borrow_refresh=args.borrow_refresh, bvh_depth=args.bvh_depth,
                        spatial_sort=not args.no_spatial_sort, scene_kind=args.scene, pool_views=args.pool_views,
                        balance_batches=args.balance_batches)
    # ---- device-timed region ------------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        sess.step(i)
        sess.settle()
    sess.sync()
    sampler.mark_begin()
    sess.reset_launch_count()
    sess.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        sess.step(args.warmup + i)
    ev1.record()
    sess.barrier()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    launches = sess.launch_count()
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    overflow = sess.settle()
    # ---- end-to-end region: public Trainer API, pinned-host inputs in, loss out, every step ------
    e2e = None
    if not args.no_e2e:
        sess.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        h2d = d2h = 0
        for i in range(args.steps):
            loss, bi, bo = sess.step_e2e(args.warmup + i)
            h2d, d2h = bi, bo
        torch.cuda.synchronize()
        sess.barrier()
        wall = time.perf_counter() - t0
        tw = torch.tensor([wall], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(tw, op=dist.ReduceOp.MAX)
        wall = float(tw.item())
        e2e = {"value": args.steps * args.batch / wall, "unit": "views/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "last_loss": loss}
    city = None
    if args.mode == "city":
        import resource

        def timed(fn):
            sess.barrier(); torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = fn()
            torch.cuda.synchronize(); sess.barrier()
            dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            return res, float(dt)

        before = sum(st.count for st in sess.stores.values())
        info, t_dens = timed(lambda: sess.densify(args.densify_threshold))
        grown = sum(st.count for st in sess.stores.values())
        rep, t_rep = timed(sess.repartition)
        for i in range(2):  # the new partition trains
            sess.step(args.warmup + i)
        after_overflow = sess.settle()
        cnt = torch.tensor([before, grown, rep["moved"], rep["after"]], dtype=torch.float64, device=device)
        mem = torch.tensor([torch.cuda.max_memory_allocated(device) / 2 ** 30,
                            resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 2 ** 20], dtype=torch.float64, device=device)
        mems = [torch.zeros_like(mem) for _ in range(world)]
        if world > 1:
            dist.all_reduce(cnt)
            dist.all_gather(mems, mem)
        else:
            mems = [mem]
        city = {"gaussians_before": int(cnt[0]), "after_densify": int(cnt[1]), "moved_by_repartition": int(cnt[2]),
                "after_repartition": int(cnt[3]), "densify_s": round(t_dens, 3), "repartition_s": round(t_rep, 3),
                "peak_device_gib_per_rank": [round(float(m[0]), 2) for m in mems],
                "peak_host_rss_gib_per_rank": [round(float(m[1]), 2) for m in mems],
                "trains_after_repartition": not after_overflow}
    # ---- eval render: composited frames through the engine's render path (the one Trainer.eval() uses) ------------
    frames = min(args.eval_frames, len(sess.cams))
    for i in range(min(2, frames)):
        sess.render_view(i)
    sess.barrier()
    torch.cuda.synchronize()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for i in range(frames):
        sess.render_view(i)
    r1.record()
    torch.cuda.synchronize()
    tr = torch.tensor([r0.elapsed_time(r1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(tr, op=dist.ReduceOp.MAX)
    render = {"ms_per_frame": float(tr) / max(frames, 1), "frames": frames,
              "what": "eval render incl. compositing across sub-models, device-timed, max over ranks"}
    phases, host_phases = None, None
    if args.phases:
        sess.engine.timer.enabled = True
        sess.engine.timer.reset()
        sess.engine.timer.trace = bool(args.trace)
        sess.engine.task_detail = bool(args.task_times)
        for i in range(args.steps):
            sess.step(args.warmup + i)
        if args.task_times:  # per-rank tables: read before the max-over-ranks reduction
            tot = sess.engine.timer.collect()
            per_rank = {k: (v if k.startswith("task.") else v / args.steps) for k, v in tot.items()}  # a task occurs once
            with open(f"{args.task_times}.rank{rank}.json", "w") as f:
                json.dump({"rank": rank, "world": world, "models": sorted(sess.stores), "ms_per_step": per_rank,
                           "relation": [[int(x) for x in row] for row in sess.relation.tolist()]}, f)
            for k in [k for k in tot if k.startswith("task.")]:  # the names differ from rank to rank: keep them out
                del sess.engine.timer.totals[k]                   # of the reduction over ranks
        host_phases = {k: round(v / args.steps, 3) for k, v in sess.engine.timer.host_totals.items() if not k.startswith("task.")}
        phases = sess.engine.timer.table(args.steps)
        if args.trace:
            sess.engine.timer.export_chrome_trace(f"{args.trace}.rank{rank}.json", rank)
        sess.engine.timer.enabled = False
    # share of this rank's Gaussians that have received a gradient so far (Adam streams only those rows)
    total_rows = sum(st.count for st in sess.stores.values())
    live_rows = round(sum(int(st.active[:st.count].sum()) for st in sess.stores.values()) / max(total_rows, 1), 4)
    roofline = None
    if phases and rank == 0:
        from retinags_b200.bench_session import phase_roofline
        peaks = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
        hbm = json.load(open(peaks)).get("hbm_gbs") if os.path.exists(peaks) else None
        roofline = phase_roofline(phases, args.batch, total_rows, sess.last_info.get("n_vis") or 0, sess.last_info.get("n_inst") or 0,
                                  int(live_rows * total_rows), args.height, args.width, sess.n_models, hbm)
    if rank == 0:
        value = args.steps * args.batch / (ms / 1e3)
        out = {
            "metric": "train views/s (62.9M GS, 1600x1036)" if (args.gaussians, args.width, args.height, args.scene) ==
            (62_900_000, 1600, 1036, "cluster") else f"train views/s ({args.gaussians / 1e6:.1f}M GS, {args.width}x{args.height})",
            "value": value, "unit": "views/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "impl": "own",
            "config": {"model": "3DGS SH-3, seeded 64-cluster mixture in a 20-unit box" if args.scene == "cluster" else
                       "3DGS SH-3, seeded aerial city scene (2000 x 2000 ground plane + building clusters)",
                       "gaussians": args.gaussians,
                       "global_batch": args.batch, "resolution": [args.width, args.height],
                       "submodels": sess.n_models, "bvh_depth": sess.bvh_depth,
                       "parallelism": f"spatial-mp{world}", "transport": sess.transport_name,
                       "border_selection_refresh_steps": sess.borrow_refresh if sess.n_models > 1 else None,
                       "l2": "inputs larger than L2 (parameter blocks of >= 1.8 GB per GPU are streamed every step)",
                       "visible_splats_per_step_rank0": sess.last_info.get("n_vis"),
                       "tile_instances_per_step_rank0": sess.last_info.get("n_inst"),
                       "rows_with_adam_moments_rank0": live_rows, "overflow_in_timed_region": overflow,
                       "two_slab_forward": os.environ.get("RGS_SLABS", "1") == "1",
                       "occlusion_culling_between_submodels": bool(sess.engine.occlusion),
                       "rows_in_morton_order": not args.no_spatial_sort,
                       "batches": ("balanced pairs" if args.balance_batches else "shuffled") + f" from {args.pool_views} cameras"
                       if args.pool_views else "consecutive cameras"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "render": render, "city": city,
            "phases_ms_per_step_max_over_ranks": phases,
            "phases_host_ms_per_step_rank0": host_phases if phases else None,
            "roofline_rank0_of_measured": roofline,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_own_trainer(args):
    """The own arm through its public trainer (``main.py``'s ``Trainer``) on the scene that the reference arm reads."""
    import torch
    import torch.distributed as dist

    from baseline import reference_arm
    from retinags_b200.config import build_parser
    from retinags_b200.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    mode = args.mode
    if mode == "trainer":
        n_train, n_test = (args.warmup + args.steps + 3) * args.batch, 2
    else:
        n_train, n_test = args.train_views, args.eval_frames
    err = ""
    if rank == 0:
        try:
            reference_arm.ensure_scene(args, n_train, n_test)
        except RuntimeError as exc:
            err = str(exc)
    if world > 1:
        box = [err]
        dist.broadcast_object_list(box, src=0)
        err = box[0]
    if err:
        raise SystemExit(err)
    root = reference_arm.scene_root(args, n_train, n_test)
    data_dir = os.path.join(root, "data")
    model_dir = os.path.join(root, f"own_model_{mode}_{world}")
    if rank == 0:  # the initial model, shared with the reference arm, under this run's own model directory
        import shutil
        shutil.rmtree(model_dir, ignore_errors=True)
        os.makedirs(os.path.join(model_dir, "point_cloud", "iteration_1"))
        os.symlink(os.path.join(root, "model", "point_cloud", "iteration_1", "point_cloud.ply"),
                   os.path.join(model_dir, "point_cloud", "iteration_1", "point_cloud.ply"))
    if world > 1:
        dist.barrier()
    depth = max(0, world.bit_length() - 1) if args.bvh_depth is None else args.bvh_depth
    max_load = args.batch * max(2, (2 ** depth + world - 1) // world)
    argv = ["-s", data_dir, "-m", model_dir, "--bvh_depth", str(depth), "--MAX_BATCH_SIZE", str(args.batch), "--MAX_LOAD",
            str(max_load), "-r", "1", "--ply_iteration", "1", "--eval", "--densify_from_iter", "100000000",
            "--DATALOADER_FIX_SEED", "--quiet", "--EVAL_INTERVAL_EPOCH", "100000", "--SAVE_INTERVAL_EPOCH", "100000",
            "--epochs", str(args.epochs if mode == "train-psnr" else 1), "--transport", {"nccl": "dist"}.get(args.transport, args.transport),
            "--BORROW_REFRESH_INTERVAL", str(args.borrow_refresh)]
    if mode == "eval":
        argv.append("--EVAL_ONLY")
    parser, lp, op, pp = build_parser()
    a = parser.parse_args(argv)
    if args.occlusion is not None:
        os.environ["RGS_OCCLUSION"] = str(args.occlusion)
    tr = Trainer(a, lp.extract(a), op.extract(a), pp.extract(a))
    out = {"impl": "own", "n_gpus": world, "mode": mode, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "fp32", "data": "synthetic", "train_views": n_train, "eval_frames": n_test,
           "config": {"model": "3DGS SH-3, seeded 64-cluster mixture in a 20-unit box", "gaussians": args.gaussians,
                      "global_batch": args.batch, "resolution": [args.width, args.height], "bvh_depth": depth,
                      "parallelism": f"spatial-mp{world}", "transport": type(tr.engine.transport).__name__}}
    from retinags_b200.ops import native
    if mode == "trainer":
        marks = {}

        def hook(step):  # device-synchronised stamps around exactly K steps, after W warm-up steps
            if step in (args.warmup, args.warmup + args.steps):
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                    torch.cuda.synchronize()
                marks[step] = (time.perf_counter(), native.launch_count())
        tr.step_callback = hook
        tr.opt.epochs = 1
        tr.train()
        (t0, l0), (t1, l1) = marks[args.warmup], marks[args.warmup + args.steps]
        sec = torch.tensor([t1 - t0], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(sec, op=dist.ReduceOp.MAX)
        sec = float(sec)
        out.update({"metric": "train views/s through Trainer.train() (scene on disk, image decoding included)",
                    "value": args.steps * args.batch / sec, "unit": "views/s", "steps": args.steps, "warmup": args.warmup,
                    "ms_per_step": 1e3 * sec / args.steps, "gpu_launches": l1 - l0})
    else:
        if mode == "train-psnr":
            tr.train()     # evaluates after its last epoch, like the reference; evaluated again below for the stamps
        res = tr.eval()
        stamps = [t for name, t in tr.eval_stamps if name == "test"]
        ms_frame = None
        if len(stamps) > 3:
            skip = min(len(stamps) - 2, 2)
            ms_frame = 1e3 * (stamps[-1] - stamps[skip - 1]) / (len(stamps) - skip)
        ev = dict(res["test"])
        ev["ms_per_frame"] = ms_frame
        out.update({"metric": "render ms/frame and PSNR (own eval loop)" if mode == "eval" else
                    f"PSNR after {args.epochs} epochs over {n_train} views (own trainer)",
                    "value": ms_frame if mode == "eval" else ev["psnr"], "unit": "ms/frame" if mode == "eval" else "dB",
                    "higher_is_better": mode != "eval", "eval": ev, "epochs": args.epochs,
                    "gpu_launches": native.launch_count()})
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_push(args):
    """Isolates the fused push of the blend epilogue: every rank renders its sub-model for one view and then repeats
    the blend kernel alone, first without destinations, then storing every row into the slot of the rank that owns it
    (peer-mapped memory), all ranks at the same time. Roofline of the fused kernel: the slower of the blend itself and
    the bytes that must leave this GPU over NVLink at the measured peer-copy bandwidth (770 GB/s per direction)."""
    import torch
    import torch.distributed as dist

    from retinags_b200.bench_session import BenchSession
    from retinags_b200.ops import native
    from retinags_b200.ops.rasterize import make_camera

    world, rank, local_rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--mode push needs >= 2 ranks (torch.distributed.run --nproc-per-node N)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    os.environ["RGS_SLABS"] = "0"  # one blend launch per render: the same launch is repeated with and without the push
    sess = BenchSession(device=device, rank=rank, world=world, n_gaussians=args.gaussians, width=args.width, height=args.height,
                        batch=1, n_views=2, gt_gaussians=min(args.gt_gaussians, 1_000_000), transport="peer", seed=args.seed,
                        borrow_refresh=args.borrow_refresh, bvh_depth=args.bvh_depth)
    eng, tr = sess.engine, sess.engine.transport
    cams, rel = sess._batch(0)
    plans = eng.plan(cams, rel)
    eng._prepare_transport(plans)
    if eng.borrow is not None:
        eng.borrow.refresh(eng.stores, need_grads=False)
    p, cam = plans[0], cams[0]
    mine = [m for m, r in zip(p.models, p.ranks) if r == rank]
    reps = max(20, args.steps)
    rows = []
    for m in mine[:1]:
        st = eng.stores[m]
        c = make_camera(cam, sess.sh_degree, st.box_lo, st.box_hi, raw_params=True, tight_rect=eng.tight_rect)
        task = eng._task(p.view, m)
        task.slabs = False
        task.forward(c, eng._segments(m, False), check=True)
        push = tr.push_plan(p, m)
        remote_bytes = sum((e[1] - e[0]) * p.W * 16 for o, e in enumerate(tr._plan_ext(p)) if o != rank and e[1] > e[0])

        def loop(with_push):
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                if with_push:
                    native.call("blend_fwd_push", device, c, task.ranges, task.vals, task.splats, task.out, None, task.n_contrib,
                                task.counters, push[0], push[1], push[2], push[3])
                else:
                    native.call("blend_fwd", device, c, task.ranges, task.vals, task.splats, task.out, None, task.n_contrib,
                                task.counters)
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps

        for _ in range(3):
            loop(True)
        t0, t1 = loop(False), loop(True)
        rows.append((t0, t1, remote_bytes))
    tr._signal_wait()
    torch.cuda.synchronize()
    tr.check()
    t0, t1, nbytes = rows[0] if rows else (0.0, 0.0, 0)
    stat = torch.tensor([t0, t1, float(nbytes)], dtype=torch.float64, device=device)
    allst = [torch.zeros_like(stat) for _ in range(world)]
    dist.all_gather(allst, stat)
    if rank == 0:
        per = [[float(x) for x in s_.tolist()] for s_ in allst]
        link = 770e9
        frac = [max(a, nb / link * 1e3) / b if b > 0 else None for a, b, nb in per]
        out = {"impl": "own", "mode": "push", "n_gpus": world, "metric": "blend kernel with the fused push vs its roofline",
               "unit": "fraction of roofline (min over ranks)", "value": min(f for f in frac if f is not None),
               "higher_is_better": True, "repeats": reps, "resolution": [args.width, args.height],
               "blend_ms_without_push": [round(a, 4) for a, _, _ in per], "blend_ms_with_push": [round(b, 4) for _, b, _ in per],
               "remote_bytes_per_launch": [int(nb) for _, _, nb in per],
               "link_ms_at_770GBs": [round(nb / link * 1e3, 4) for _, _, nb in per],
               "fraction_of_roofline": [round(f, 3) if f is not None else None for f in frac],
               "roofline": "max(blend without push, remote bytes / 770 GB/s measured peer copy) / blend with push",
               "config": {"gaussians": args.gaussians, "submodels": sess.n_models}}
        print(json.dumps(out), flush=True)
    dist.barrier()
    tr.close()
    dist.destroy_process_group()


def run_reference(args):
    from baseline import reference_arm
    reference_arm.main(args)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    elif a.mode == "push":
        run_push(a)
    elif a.mode not in ("train", "city"):
        run_own_trainer(a)
    else:
        run_own(a)
