"""Configuration groups and the command-line surface.

Same flags as the reference (``arguments/__init__.py:19-137`` for the three parameter groups,
``main.py:73-116`` for the trainer flags): a ``ParamGroup`` registers ``--name`` (and ``-n`` for
underscore-prefixed fields) for every attribute, booleans become ``store_true``.
"""
from __future__ import annotations

from argparse import ArgumentParser, Namespace


class ParamGroup:
    def __init__(self, parser: ArgumentParser, name: str, fill_none: bool = False):
        group = parser.add_argument_group(name)
        for key, value in vars(self).items():
            shorthand = key.startswith("_")
            if shorthand:
                key = key[1:]
            t = type(value)
            value = value if not fill_none else None
            names = ["--" + key] + (["-" + key[0]] if shorthand else [])
            if t == bool:
                group.add_argument(*names, default=value, action="store_true")
            else:
                group.add_argument(*names, default=value, type=t)

    def extract(self, args) -> Namespace:
        out = Namespace()
        for k, v in vars(args).items():
            if k in vars(self) or ("_" + k) in vars(self):
                setattr(out, k, v)
        return out


class ModelParams(ParamGroup):
    def __init__(self, parser, sentinel: bool = False):
        self.sh_degree = 3
        self._source_path = ""
        self._model_path = ""
        self._images = "images"
        self._resolution = -1
        self._white_background = False
        self.data_device = "cuda"
        self.eval = False
        self.scale_control_rate = 1.0
        self.opacity_init = 0.1
        self.pointcloud_sample_rate = 1
        self.points3D = "points3D"
        self.without_normal = False
        super().__init__(parser, "Loading Parameters", sentinel)


class PipelineParams(ParamGroup):
    def __init__(self, parser):
        self.convert_SHs_python = False
        self.compute_cov3D_python = False
        self.debug = False
        self.max_batch_size = 1
        self.max_load = 2
        self.render_version = "default"
        super().__init__(parser, "Pipeline Parameters")


class OptimizationParams(ParamGroup):
    def __init__(self, parser):
        self.iterations = 30_000
        self.epochs = -1
        self.position_lr_init = 0.00016
        self.position_lr_final = 0.0000016
        self.position_lr_delay_mult = 0.01
        self.position_lr_max_steps = 30_000
        self.scaling_lr = 0.005
        self.scaling_lr_init = 0.005
        self.scaling_lr_final = 0.005
        self.scaling_lr_delay_mult = 0.01
        self.scaling_lr_max_steps = 30_000
        self.feature_lr = 0.0025
        self.opacity_lr = 0.05
        self.rotation_lr = 0.001
        self.percent_dense = 0.01
        self.lambda_dssim = 0.2
        self.densification_interval = 100
        self.opacity_reset_interval = 3000
        self.densify_from_iter = 500
        self.densify_until_iter = 15_000
        self.densify_grad_threshold = 0.0002
        self.random_background = False
        # parsed for command-line compatibility; unused by the trainer (as in the reference)
        self.lambda_perception = 0.0
        self.scales_reg_2d = 0.0
        self.scales_reg_3d = 0.0
        self.huber_delta = 0.0
        self.max_gaussians = 0
        self.screen_size_threshold = 20
        self.densify_epoch_interval = 0
        self.opacity_reset_epoch_interval = 0
        super().__init__(parser, "Optimization Parameters")


def add_trainer_flags(parser: ArgumentParser):
    """Flags of the reference's ``main.py:77-114``."""
    p = parser
    p.add_argument("--detect_anomaly", action="store_true", default=False)
    p.add_argument("--test_iterations", nargs="+", type=int, default=[])
    p.add_argument("--SPLIT_MODEL", action="store_true", default=False)
    p.add_argument("--quiet", action="store_true")
    p.add_argument("--checkpoint_iterations", nargs="+", type=int, default=[])
    p.add_argument("--bvh_depth", type=int, default=2, help="2^bvh_depth sub-models")
    p.add_argument("--logdir", type=str, default="./tf_logs/")
    p.add_argument("--ply_iteration", type=int, default=-1)
    p.add_argument("--CKPT_MAX_NUM", type=int, default=5)
    p.add_argument("--ENABLE_REPARTITION", action="store_true", default=False)
    p.add_argument("--REPARTITION_START_EPOCH", type=int, default=10)
    p.add_argument("--REPARTITION_END_EPOCH", type=int, default=300)
    p.add_argument("--REPARTITION_INTERVAL_EPOCH", type=int, default=50)
    p.add_argument("--EVAL_PSNR_INTERVAL", type=int, default=8)
    p.add_argument("--Z_NEAR", type=float, default=0.01)
    p.add_argument("--Z_FAR", type=float, default=1000.0)
    p.add_argument("--EVAL_INTERVAL_EPOCH", type=int, default=5)
    p.add_argument("--SAVE_INTERVAL_EPOCH", type=int, default=100000)
    p.add_argument("--SAVE_INTERVAL_ITER", type=int, default=50000)
    p.add_argument("--SKIP_PRUNE_AFTER_RESET", type=int, default=0)
    p.add_argument("--SKIP_SPLIT", action="store_true", default=False)
    p.add_argument("--SKIP_CLONE", action="store_true", default=False)
    p.add_argument("--NOT_SHRAE_GS_INFO", action="store_true", default=False)
    p.add_argument("--MAX_SIZE_SINGLE_GS", type=int, default=int(1e7))
    p.add_argument("--MAX_BATCH_SIZE", type=int, default=4)
    p.add_argument("--MAX_LOAD", type=int, default=16)
    p.add_argument("--ENABLE_TENSORBOARD", action="store_true", default=False)
    p.add_argument("--EVAL_ONLY", action="store_true", default=False)
    p.add_argument("--SAVE_EVAL_IMAGE", action="store_true", default=False)
    p.add_argument("--SAVE_EVAL_SUB_IMAGE", action="store_true", default=False)
    p.add_argument("--USE_RELATION_CACHE", action="store_true", default=False)
    p.add_argument("--log_level", type=int, default=20)
    p.add_argument("--DATALOADER_FIX_SEED", action="store_true", default=False)
    # additions of this framework
    p.add_argument("--transport", default="auto", choices=["auto", "peer", "dist", "local"],
                   help="partial-image transport: fused peer-to-peer stores, torch.distributed send/recv, or local")
    p.add_argument("--device", default="auto", choices=["auto", "cuda", "cpu"])
    p.add_argument("--synthetic", default="", help="name of a seeded synthetic scene instead of -s (see data/synthetic.py)")
    p.add_argument("--WATCHDOG_TIMEOUT", type=float, default=120.0,
                   help="seconds without a heartbeat after which a peer counts as failed (0 disables the watchdog)")
    p.add_argument("--LPIPS_WEIGHTS", default="", help="directory with vgg16.pth and lpips_vgg.pth; without it LPIPS is NaN")
    p.add_argument("--COMM_VERSION", default="0", choices=["0", "0+profiling", "1", "2"],
                   help="schedule of the torch.distributed transport: batched, batched inside a profiler range, blocking "
                        "in rank order, two-pass isend/irecv")
    p.add_argument("--BALANCE_BATCHES", action="store_true", default=False,
                   help="batch cameras whose estimated per-rank loads complement each other (same cameras per epoch)")
    p.add_argument("--BORROW_REFRESH_INTERVAL", type=int, default=8,
                   help="steps between recomputations of the border-Gaussian sets; the rows are re-sent every step, the "
                        "sets are made 5 %% larger when they are kept (1 = recomputed every step, as the reference)")
    p.add_argument("--PREFETCH_BATCHES", type=int, default=2,
                   help="batches decoded ahead of the step per decoding thread (the reference's prefetch_factor); 0 decodes "
                        "in the training thread")
    p.add_argument("--PREFETCH_WORKERS", type=int, default=8, help="threads decoding images for the coming batches")
    p.add_argument("--OCCLUSION_CULLING", type=int, default=-1, choices=[-1, 0, 1],
                   help="skip tiles that nearer sub-models have finished (maps exchanged once per step); -1: the default "
                        "of the build (RGS_OCCLUSION)")
    p.add_argument("--SPATIAL_SORT", type=int, default=1, choices=[0, 1],
                   help="keep the rows of every sub-model in Morton order of their positions (re-sorted after load, "
                        "densification and repartition)")
    p.add_argument("--MODEL_ASSIGNMENT", default="round_robin", choices=["round_robin", "cost"],
                   help="sub-model -> rank map: i %% world as the reference, or balanced by the estimated render cost over "
                        "the training cameras")


def build_parser() -> tuple[ArgumentParser, ModelParams, OptimizationParams, PipelineParams]:
    parser = ArgumentParser(description="Model-parallel 3D Gaussian Splatting trainer (B200)")
    lp, op, pp = ModelParams(parser), OptimizationParams(parser), PipelineParams(parser)
    add_trainer_flags(parser)
    return parser, lp, op, pp


def get_combined_args(parser: ArgumentParser, argv=None) -> Namespace:
    """Command line merged over the ``cfg_args`` file of ``--model_path`` (``arguments/__init__.py:139-159``): values
    given on the command line win. The file holds a ``Namespace(...)`` literal; it is parsed, never evaluated."""
    import ast
    import os
    import sys
    args_cmd = parser.parse_args(sys.argv[1:] if argv is None else argv)
    merged = {}
    path = os.path.join(args_cmd.model_path or "", "cfg_args")
    if os.path.exists(path):
        text = open(path).read().strip()
        call = ast.parse(text, mode="eval").body
        if isinstance(call, ast.Call) and getattr(call.func, "id", "") == "Namespace":
            merged = {kw.arg: ast.literal_eval(kw.value) for kw in call.keywords}
    for k, v in vars(args_cmd).items():
        if v is not None or k not in merged:
            merged[k] = v
    return Namespace(**merged)
