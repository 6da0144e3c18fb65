"""Model-parallel trainer / evaluator.

Public API mirrors the reference's ``Trainer4TreePartition`` (``parallel_utils/basic_parallel_trainer/
trainer4tree_partition.py:42-777``): ``Trainer(args, mdp, opt, pipe)``, ``.train()``, ``.eval()``.  One
process per GPU (or per CPU rank with gloo); the Gaussians are cut by a kd/BVH tree over a 2048x2048x1
load grid into ``2^bvh_depth`` sub-models, sub-model ``i`` lives on rank ``i % world``; a step renders
every visible local sub-model, composites the partial images in front-to-back order on row bands spread
over the ranks, evaluates L1 + D-SSIM, and sends gradients back.

Checkpoint layout (``-m`` root; same as the reference, ``scene_utils.py:123-140``,
``trainer4tree_partition.py:673-679``)::

    <m>/rank_<r>/point_cloud/iteration_<it>/point_cloud_<mid>.ply   adam_<mid>.pt   tree_<r>.txt
    <m>/rank_<r>/cameras.json  trainset_relation.pt  testset_relation.pt  rank_<r>_<time>.txt
    <m>/point_cloud/iteration_<it>/point_cloud.ply                   merged vanilla-3DGS model
    <m>/img/<split>_<name>_<it>.png   <m>/gt/<name>.png

Behavioural choices where the reference is ambiguous or broken are stated where they are made
(``_repartition``: the relation matrices are recomputed without the reference's missing argument;
exceptions propagate with a non-zero exit instead of being swallowed, ``main.py:66-68``).
"""
from __future__ import annotations

import glob
import json
import logging
import os
import shutil
import time

import numpy as np
import torch
import torch.distributed as dist

from .data import readers
from .data.cameras import Camera
from .data.datasets import CameraListDataset, DatasetRepeater
from .data.prefetch import BatchPrefetcher
from .engine import StepEngine
from .models import densify, ply_io
from .models.gaussians import GaussianStore
from .ops.knn import knn3_dist2
from .parallel.balancer import WorkloadBalancer
from .parallel.border import BorderExchange
from .parallel.compositing import LocalTransport, TorchDistTransport
from .parallel.partition import BvhTree, Grid3D, assign_models, load_histogram
from .utils.general import expon_lr, inverse_sigmoid, is_interval_in_batch, is_point_in_batch
from .utils.image import psnr_from_mse, save_png

from .utils.sh import RGB2SH as rgb_to_sh  # noqa: E402


class CkptCleaner:
    """Keep the newest ``max_len`` checkpoint folders (``scene_utils.py:105-121``)."""

    def __init__(self, max_len: int = 5):
        self.buf, self.max_len = [], max_len

    def add(self, folder: str):
        if folder in self.buf:
            return
        self.buf.append(folder)
        while len(self.buf) > self.max_len:
            shutil.rmtree(self.buf.pop(0), ignore_errors=True)


class Trainer:
    SCENE_GRID_SIZE = (2048, 2048, 1)
    SPLIT_ORDERS = (0, 1)

    def __init__(self, args, mdp, opt, pipe, group=None, scene: readers.SceneInfo | None = None):
        self.args, self.mdp, self.opt, self.pipe, self.group = args, mdp, opt, pipe, group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        want = getattr(args, "device", "auto")
        use_cuda = torch.cuda.is_available() and want != "cpu"
        self.device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
        self.bvh_depth = args.bvh_depth
        if self.world > 2 ** self.bvh_depth:
            raise ValueError(f"WORLD_SIZE {self.world} exceeds the number of sub-models 2^{self.bvh_depth}")
        self.sh_degree = mdp.sh_degree
        self.model_root = mdp.model_path
        self.model_path = os.path.join(self.model_root, f"rank_{self.rank}")
        os.makedirs(self.model_path, exist_ok=True)
        self._init_logging()
        self.cleaner = CkptCleaner(args.CKPT_MAX_NUM)
        # ---- scene ----------------------------------------------------------------------------------
        self.scene = scene if scene is not None else readers.read_scene(
            mdp.source_path, mdp.images, mdp.eval, mdp.points3D, mdp.pointcloud_sample_rate)
        self.cameras_extent = float(self.scene.nerf_normalization["radius"])
        self.train_dataset = CameraListDataset(self.scene.train_cameras, mdp.resolution, 1.0, mdp.white_background)
        self.test_dataset = CameraListDataset(self.scene.test_cameras, mdp.resolution, 1.0, mdp.white_background)
        self.background = (1.0, 1.0, 1.0) if mdp.white_background else (0.0, 0.0, 0.0)
        if self.rank == 0:
            cams = [self.test_dataset.empty_item(i) for i in range(len(self.test_dataset))] + \
                   [self.train_dataset.empty_item(i) for i in range(len(self.train_dataset))]
            json.dump([c.to_json(i) for i, c in enumerate(cams)], open(os.path.join(self.model_path, "cameras.json"), "w"))
        os.makedirs(os.path.join(self.model_root, "img"), exist_ok=True)
        os.makedirs(os.path.join(self.model_root, "gt"), exist_ok=True)
        # ---- model ----------------------------------------------------------------------------------
        self.whole_mode = not args.SPLIT_MODEL
        self.load_iteration = args.ply_iteration if args.ply_iteration > 0 else self._find_iteration()
        self.iteration = max(self.load_iteration, 0)
        self.stores: dict[int, GaussianStore] = {}
        self._init_partition_and_models()
        # ---- engine -----------------------------------------------------------------------------------
        self._build_engine()
        self.train_rlt = self._relation(self.train_dataset, "trainset_relation.pt")
        self.test_rlt = self._relation(self.test_dataset, "testset_relation.pt")
        self._gen = torch.Generator(device=self.device)
        self._gen.manual_seed(1234 + self.rank)
        self.steps_done = 0         # training steps (batches) run by this object
        self.step_callback = None   # optional callable(step index), called before each training step (benchmarks)
        self.eval_stamps: list = []  # (split, host time after the metrics of an image were read) of the last eval()
        self.watchdog = None
        if self.world > 1 and getattr(args, "WATCHDOG_TIMEOUT", 120.0) > 0:
            from .parallel.watchdog import Watchdog
            try:
                base = dist.distributed_c10d._get_default_store()
                self.watchdog = Watchdog(dist.PrefixStore("rgs_watchdog", base), self.rank, self.world, interval=2.0,
                                         timeout=float(getattr(args, "WATCHDOG_TIMEOUT", 120.0))).start()
            except Exception as exc:  # a backend without a reachable store: run without host heartbeats
                self.logger.warning("watchdog disabled: %r", exc)

    # ------------------------------------------------------------------------------------------------
    # set-up helpers
    # ------------------------------------------------------------------------------------------------
    def _init_logging(self):
        self.logger = logging.getLogger(f"rank_{self.rank}")
        self.logger.setLevel(getattr(self.args, "log_level", 20))
        self.logger.propagate = False
        stamp = time.strftime("%Y_%m_%d_%H_%M_%S", time.localtime())
        fh = logging.FileHandler(os.path.join(self.model_path, f"rank_{self.rank}_{stamp}.txt"), mode="w")
        fh.setFormatter(logging.Formatter("%(asctime)s-%(filename)s[line:%(lineno)d]-%(levelname)s: %(message)s"))
        self.logger.handlers = [fh]
        self.tb = None
        if getattr(self.args, "ENABLE_TENSORBOARD", False):
            try:
                from torch.utils.tensorboard import SummaryWriter
                logdir = os.path.join(self.args.logdir, f"rank_{self.rank}") if self.args.logdir else self.model_path
                self.tb = SummaryWriter(logdir)
            except ImportError:
                self.logger.warning("tensorboard not available")

    def _bcast(self, obj):
        if self.world == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]

    def _barrier(self):
        if self.world > 1:
            dist.barrier(self.group)

    def _find_iteration(self) -> int:
        base = self.model_root if self.whole_mode else self.model_path
        its = []
        for d in glob.glob(os.path.join(base, "point_cloud", "iteration_*")):
            try:
                its.append(int(os.path.basename(d).split("_")[-1]))
            except ValueError:
                pass
        return max(its) if its else 0

    def _stores_from_tree(self):
        lo, hi = self.tree.leaf_boxes_world(open_border=True)
        self.n_models = len(self.tree.leaves)
        self.model2rank = assign_models(self.n_models, self.world, self._assignment_costs())
        self.local_ids = [m for m in range(self.n_models) if self.model2rank[m] == self.rank]
        if not self.local_ids:
            raise RuntimeError("empty rank")
        self.boxes = (lo, hi)
        return lo, hi

    def _assignment_costs(self):
        """Per sub-model cost for ``--MODEL_ASSIGNMENT cost``: how many training cameras see its box (the median
        split already gives every leaf the same number of points). None keeps the reference's i % world."""
        if getattr(self.args, "MODEL_ASSIGNMENT", "round_robin") != "cost" or self.n_models <= self.world:
            return None
        costs = None
        if self.rank == 0:
            ds = self.train_dataset
            cams = [ds.empty_item(i) for i in range(len(ds))]
            rel = self.tree.relation(cams, self.args.Z_NEAR, self.args.Z_FAR)
            costs = [float(c) + 1.0 for c in (rel >= 0).sum(0)]
        return self._bcast(costs)

    def _init_partition_and_models(self):
        a = self.args
        rng = np.random.default_rng(0)
        if self.load_iteration > 0 and not self.whole_mode:
            tree_file = os.path.join(self.model_root, "rank_0", "point_cloud", f"iteration_{self.load_iteration}", "tree_0.txt")
            self.tree = BvhTree.load(tree_file)
            lo, hi = self._stores_from_tree()
            for m in self.local_ids:
                found = glob.glob(os.path.join(self.model_root, "rank_*", "point_cloud", f"iteration_{self.load_iteration}",
                                               f"point_cloud_{m}.ply"))
                if not found:
                    raise FileNotFoundError(f"point_cloud_{m}.ply of iteration {self.load_iteration}")
                g = ply_io.load_gaussians(found[0], self.sh_degree)
                st = GaussianStore(g["xyz"].shape[0], self.device, self.sh_degree, lo[m], hi[m], m)
                st.set_params(g)
                adam = os.path.join(os.path.dirname(found[0]), f"adam_{m}.pt")
                if os.path.exists(adam):
                    st.load_optimizer_state_dict(torch.load(adam, map_location="cpu", weights_only=False))
                self.stores[m] = st
        elif self.load_iteration > 0:
            ply = os.path.join(self.model_root, "point_cloud", f"iteration_{self.load_iteration}", "point_cloud.ply")
            self._load_whole_model(ply, rng)
        else:
            pts, col = self.scene.points, self.scene.colors
            if pts is None:
                raise ValueError("no initial point cloud")
            grid = Grid3D.from_points(pts.astype(np.float64), self.SCENE_GRID_SIZE)
            grid.accumulate(pts)
            self.tree = BvhTree.build(grid, self.bvh_depth, self.SPLIT_ORDERS, rng=rng)
            lo, hi = self._stores_from_tree()
            flo, fhi = self.tree.leaf_boxes_world(open_border=False)
            p = torch.from_numpy(pts.astype(np.float32))
            c = torch.from_numpy(col.astype(np.float32))
            ids = self.tree.label(p)
            for m in self.local_ids:
                sel = (ids == m).nonzero(as_tuple=True)[0]
                self.stores[m] = self._create_from_points(p[sel], c[sel], lo[m], hi[m], m)
        active = min(self.sh_degree, self.iteration // 1000) if self.load_iteration > 0 else 0
        self._spatial_sort()
        for st in self.stores.values():
            st.active_sh_degree = active
        self.logger.info("sub-models %s on rank %d: %s", self.local_ids, self.rank, {m: s.count for m, s in self.stores.items()})

    LOAD_CHUNK_ROWS = 2_000_000

    def _load_whole_model(self, ply: str, rng):
        """Start from one whole-model file of any size. The file is memory-mapped and walked in chunks, never parsed
        as a whole (the reference parses it into host memory on rank 0 and scatters it with point-to-point messages,
        ``gaussian_utils.py:128-171``, ``gaussian_nn_module.py:134-261``):

        1. every rank scans a 1/world share of the chunks for the bounds (positions +- 3 max scale) and, after the
           bounds are agreed, for the load histogram; both are all-reduced; rank 0 builds the tree and broadcasts it;
        2. every rank walks all chunks once and keeps the Gaussians of its own sub-models.

        No rank holds more than one chunk besides its own sub-models. With ``--NOT_SHRAE_GS_INFO`` a sub-model keeps
        every Gaussian whose 3-sigma extent reaches its box instead of only those whose centre lies in it, because no
        border Gaussians are exchanged afterwards (``gaussian_utils.py:177-193``, ``gaussian_nn_module.py:1028-1036``)."""
        a = self.args
        rows = self.LOAD_CHUNK_ROWS
        stream = ply_io.PlyVertexStream(ply)
        lo = torch.full((3,), float("inf"), dtype=torch.float64)
        hi = torch.full((3,), float("-inf"), dtype=torch.float64)
        smax = torch.zeros(1, dtype=torch.float64)
        for _, v in stream.chunks(rows, self.rank, self.world):
            xyz = torch.from_numpy(np.stack([v["x"], v["y"], v["z"]], 1).astype(np.float64))
            sc = np.stack([v[n] for n in stream.names if n.startswith("scale_")], 1).astype(np.float64)
            lo, hi = torch.minimum(lo, xyz.min(0).values), torch.maximum(hi, xyz.max(0).values)
            smax = torch.maximum(smax, torch.from_numpy(np.exp(sc.max(keepdims=True)).reshape(1)))
        if self.world > 1:
            pack = torch.cat([-lo, hi, smax]).to(self.device)  # one MAX reduction for all three
            dist.all_reduce(pack, op=dist.ReduceOp.MAX, group=self.group)
            pack = pack.cpu()
            lo, hi, smax = -pack[:3], pack[3:6], pack[6:]
        ext = 3.0 * float(smax)
        grid = Grid3D((lo - ext).numpy(), (hi + ext).numpy(), self.SCENE_GRID_SIZE)
        for _, v in stream.chunks(rows, self.rank, self.world):
            grid.accumulate(np.stack([v["x"], v["y"], v["z"]], 1).astype(np.float32))
        if self.world > 1:
            load = torch.from_numpy(np.ascontiguousarray(grid.load)).to(self.device)
            dist.all_reduce(load, group=self.group)
            grid.load = load.cpu().numpy()
        self.tree = self._bcast(BvhTree.build(grid, self.bvh_depth, self.SPLIT_ORDERS, rng=rng) if self.rank == 0 else None)
        blo, bhi = self._stores_from_tree()
        for m in self.local_ids:
            self.stores[m] = GaussianStore(max(stream.count // max(self.n_models, 1), 4), self.device, self.sh_degree,
                                           blo[m], bhi[m], m)
        keep_reach = bool(a.NOT_SHRAE_GS_INFO)
        for _, g in ply_io.iter_gaussians(ply, self.sh_degree, rows):
            if keep_reach:
                r = 3.0 * torch.exp(g["scale"]).max(dim=1, keepdim=True).values
                for m in self.local_ids:
                    mlo = torch.as_tensor(blo[m], dtype=torch.float32)
                    mhi = torch.as_tensor(bhi[m], dtype=torch.float32)
                    sel = ((g["xyz"] + r >= mlo) & (g["xyz"] - r <= mhi)).all(dim=1).nonzero(as_tuple=True)[0]
                    if sel.numel():
                        self.stores[m].append_new({k: v[sel].to(self.device) for k, v in g.items()})
            else:
                ids = self.tree.label(g["xyz"])
                for m in self.local_ids:
                    sel = (ids == m).nonzero(as_tuple=True)[0]
                    if sel.numel():
                        self.stores[m].append_new({k: v[sel].to(self.device) for k, v in g.items()})

    def _spatial_sort(self):
        if getattr(self.args, "SPATIAL_SORT", 1):
            for st in self.stores.values():
                st.spatial_sort()

    def _create_from_points(self, pts: torch.Tensor, rgb: torch.Tensor, lo, hi, mid: int) -> GaussianStore:
        """3DGS initialisation per sub-model (``scene/gaussian_nn_module.py:403-427``): SH DC from the point
        colours, isotropic scale from the mean distance to the 3 nearest neighbours *inside the sub-model*."""
        n = pts.shape[0]
        st = GaussianStore(max(n, 4), self.device, self.sh_degree, lo, hi, mid)
        if n == 0:
            return st
        p = pts.to(self.device)
        d2 = torch.clamp_min(knn3_dist2(p), 1e-7)
        scale = torch.log(torch.sqrt(d2) * self.mdp.scale_control_rate)[:, None].repeat(1, 3)
        sh = torch.zeros(n, 16, 3, device=self.device)
        sh[:, 0] = rgb_to_sh(rgb.to(self.device))
        rot = torch.zeros(n, 4, device=self.device)
        rot[:, 0] = 1
        opacity = inverse_sigmoid(self.mdp.opacity_init * torch.ones(n, 1, device=self.device))
        st.set_params(dict(xyz=p, sh=sh.view(n, 48), scale=scale, rot=rot, opacity=opacity))
        return st

    def _close_engine(self):
        """Release the peer-mapped regions of the current engine (collective with the peer transport)."""
        if getattr(self, "border", None) is not None and hasattr(self.border, "close"):
            self.border.close()
        eng = getattr(self, "engine", None)
        if eng is not None and hasattr(eng.transport, "close"):
            eng.transport.close()

    def _build_engine(self):
        a = self.args
        kind = getattr(a, "transport", "auto")
        if self.world == 1 or kind == "local":
            tr = LocalTransport(self.device)
        elif kind in ("auto", "peer") and self.device.type == "cuda":
            try:
                from .parallel.peer import PeerTransport
                tr = PeerTransport(self.device, self.group, max_views=max(a.MAX_BATCH_SIZE, 1))
            except Exception as exc:
                if kind == "peer":
                    raise
                self.logger.warning("peer transport unavailable (%r); using torch.distributed send/recv", exc)
                tr = TorchDistTransport(self.device, self.group, getattr(a, "COMM_VERSION", "0"))
        else:
            tr = TorchDistTransport(self.device, self.group, getattr(a, "COMM_VERSION", "0"))
        lo, hi = self.boxes
        self.border = None
        if self.n_models > 1 and not a.NOT_SHRAE_GS_INFO:
            interval = getattr(a, "BORROW_REFRESH_INTERVAL", 1)
            if hasattr(tr, "push_plan"):
                from .parallel.peer_border import PeerBorderExchange
                self.border = PeerBorderExchange(lo, hi, self.model2rank, self.rank, self.world, self.device, tr, self.group,
                                                 interval)
            else:
                self.border = BorderExchange(lo, hi, self.model2rank, self.rank, self.world, self.device, self.group, interval)
        self.engine = StepEngine(self.stores, self.model2rank, self.device, tr, self.opt.lambda_dssim, self.background,
                                 borrow=self.border)
        if getattr(a, "OCCLUSION_CULLING", -1) >= 0:
            self.engine.occlusion = bool(a.OCCLUSION_CULLING)
        self.engine.debug = bool(getattr(self.pipe, "debug", False))
        self.engine.detect_anomaly = bool(getattr(self.args, "detect_anomaly", False))
        self.engine.dump_dir = self.model_path
        self.balancer = WorkloadBalancer(self.world, self.model2rank)

    def _relation(self, dataset: CameraListDataset, cache_name: str, use_cache: bool = True) -> np.ndarray:
        """Camera -> sub-model relation (visibility and front-to-back position) of a dataset. Rank 0 alone decides
        whether the cached file is used and every rank takes part in the one broadcast, so that all ranks follow the
        same collective path; the file is written after the broadcast. After a repartition the tree has changed while
        the shape of the matrix has not: the callers pass ``use_cache=False`` there (the reference recomputes as well,
        ``trainer4tree_partition.py:308-314``)."""
        rel = None
        if self.rank == 0:
            path = os.path.join(self.model_root, "rank_0", cache_name)
            if use_cache and self.args.USE_RELATION_CACHE and os.path.exists(path):
                cached = torch.load(path, weights_only=False)
                cached = cached.numpy() if isinstance(cached, torch.Tensor) else np.asarray(cached)
                if cached.shape == (len(dataset), self.n_models):
                    rel = cached.astype(np.int32)
            if rel is None:
                cams = [dataset.empty_item(i) for i in range(len(dataset))]
                rel = self.tree.relation(cams, self.args.Z_NEAR, self.args.Z_FAR) if cams else \
                    np.zeros((0, self.n_models), np.int32)
        rel = self._bcast(rel)
        if self.rank == 0:
            torch.save(torch.from_numpy(np.ascontiguousarray(rel)), os.path.join(self.model_path, cache_name))
        return rel

    # ------------------------------------------------------------------------------------------------
    # schedules
    # ------------------------------------------------------------------------------------------------
    def learning_rates(self, iteration: int):
        o = self.opt
        xyz = expon_lr(iteration, o.position_lr_init * self.cameras_extent, o.position_lr_final * self.cameras_extent,
                       0, o.position_lr_delay_mult, o.position_lr_max_steps)
        # the reference ties the scaling schedule to len(train)*epochs, which is negative with the default
        # --epochs -1, so the scaling rate stays at its initial value (trainer4tree_partition.py:207)
        max_steps = len(self.train_dataset) * o.epochs
        scale = o.scaling_lr if max_steps <= 0 else expon_lr(iteration, o.scaling_lr_init, o.scaling_lr_final, 0,
                                                               o.scaling_lr_delay_mult, max_steps)
        return (xyz, o.feature_lr, o.feature_lr / 20.0, scale, o.rotation_lr, o.opacity_lr)

    # ------------------------------------------------------------------------------------------------
    # training
    # ------------------------------------------------------------------------------------------------
    def _prefetch_depth(self) -> int:
        """Batches decoded ahead of the step: ``--PREFETCH_BATCHES`` per decoding thread, the reference's
        ``prefetch_factor`` x ``num_workers`` (2 x 8 batches in flight), so that every thread has an image to work on
        even when a batch is a single view. 0 decodes in the training thread."""
        a = self.args
        return max(0, int(getattr(a, "PREFETCH_BATCHES", 2))) * max(1, int(getattr(a, "PREFETCH_WORKERS", 8)))

    def _epoch_groups(self, epoch: int):
        seed = 0 if self.args.DATALOADER_FIX_SEED else epoch
        g = torch.Generator()
        g.manual_seed(seed)
        order = torch.randperm(len(self.train_dataset), generator=g).tolist()
        if getattr(self.args, "BALANCE_BATCHES", False) and self.world > 1:
            cost = self._camera_costs()
            groups = self.balancer.groups_balanced(self.train_rlt, order, cost, self.args.MAX_LOAD,
                                                   self.args.MAX_BATCH_SIZE) if self.rank == 0 else None
        else:
            groups = self.balancer.groups(self.train_rlt, order, self.args.MAX_LOAD, self.args.MAX_BATCH_SIZE) if self.rank == 0 else None
        return self._bcast(groups)

    def _camera_costs(self) -> np.ndarray:
        """Estimated tile instances per (training camera, sub-model); recomputed when the model set changed."""
        key = tuple(sorted((m, st.count) for m, st in self.stores.items()))
        if getattr(self, "_cost_key", None) != key:
            from .parallel.balancer import estimate_costs
            cams = [self.train_dataset.empty_item(i) for i in range(len(self.train_dataset))]
            cost = torch.from_numpy(estimate_costs(self.stores, cams, self.n_models)).to(self.device)
            if self.world > 1:
                dist.all_reduce(cost, group=self.group)
            self._cost, self._cost_key = cost.cpu().numpy(), key
        return self._cost

    def train(self):
        o, a = self.opt, self.args
        n_train = len(self.train_dataset)
        start_epoch = int(round(self.iteration / max(n_train, 1)))
        epochs = o.epochs if o.epochs > 0 else int(round(o.iterations / max(n_train, 1)))
        ema = None
        t_last = time.time()
        for epoch in range(start_epoch, epochs):
            groups = self._epoch_groups(epoch)
            lrs = self.learning_rates(self.iteration)
            sh_deg = min(self.sh_degree, self.iteration // 1000)
            for st in self.stores.values():
                st.active_sh_degree = sh_deg
            feed = BatchPrefetcher(self.train_dataset, groups, depth=self._prefetch_depth(),
                                   workers=getattr(a, "PREFETCH_WORKERS", 8))
            for ids, cams in feed:  # the images of the next batches are decoded while this step runs
                if self.watchdog is not None:
                    self.watchdog.check()  # a dead peer is noticed here, before the next kernels and collectives
                if self.step_callback is not None:
                    self.step_callback(self.steps_done)
                bs = len(cams)
                t0 = time.perf_counter()
                bg = None
                if o.random_background:
                    # a random background colour per step (the reference draws it in its blender when the option is
                    # set, result_aggregator.py:256); seeded by the iteration so that every rank composites with the same
                    gen = torch.Generator().manual_seed(1_000_003 + self.iteration)
                    bg = tuple(torch.rand(3, generator=gen).tolist())
                res = self.engine.train_step(cams, self.train_rlt[list(ids)], sh_deg, lrs, optimizer_step=False, background=bg)
                # after a densification the reference's rebuilt optimiser holds no gradients, so that step
                # updates nothing (trainer4tree_partition.py:657-666); same here
                if not self._densify_and_reset(self.iteration, bs):
                    self.engine.optimizer_step(lrs)
                if self.iteration % 10 < bs or self.tb:
                    loss = self._reduce_loss(res)
                    ema = loss if ema is None else 0.4 * loss + 0.6 * ema
                    if self.tb:
                        self.tb.add_scalar("train_loss_patches/total_loss", loss, self.iteration)
                        self.tb.add_scalar("iter_time", (time.perf_counter() - t0) * 1e3, self.iteration)
                        if self.device.type == "cuda":
                            self.tb.add_scalar("cnt/memory", torch.cuda.memory_allocated() / 2 ** 30, self.iteration)
                    if self.rank == 0 and not a.quiet and time.time() - t_last > 5:
                        print(f"[iter {self.iteration}] loss {ema:.6f} points {sum(s.count for s in self.stores.values())}", flush=True)
                        t_last = time.time()
                # every step, without waiting for the device: the counters of the newest step whose copies have arrived
                # (buffers grow before the next forward; a step that overflowed was dropped by the optimiser on all ranks)
                info = self.engine.poll_async()
                if info is not None and info.get("dropped"):
                    self.logger.warning("a render of the step before iteration %d ran out of instance capacity: its update "
                                        "was dropped on every rank, the buffers have been grown", self.iteration + bs)
                self.iteration += bs
                self.steps_done += 1
            last = epoch == epochs - 1
            if (epoch % a.SAVE_INTERVAL_EPOCH == 0 and epoch != 0) or last:
                self.save(self.iteration)
            if last and self.whole_mode:
                self._barrier()
                if self.rank == 0:
                    self.save_whole_model(self.iteration)
            if a.ENABLE_REPARTITION and epoch % a.REPARTITION_INTERVAL_EPOCH == 0 and \
                    a.REPARTITION_START_EPOCH <= epoch <= a.REPARTITION_END_EPOCH:
                self._repartition()
            if (epoch % a.EVAL_INTERVAL_EPOCH == 0 and epoch != 0) or last:
                self.eval()
        self.logger.info("complete")

    def _reduce_loss(self, res) -> float:
        if not res.sums:
            return 0.0
        s = torch.stack(res.sums)
        if self.world > 1:
            dist.all_reduce(s, group=self.group)
        total = 0.0
        lam = self.opt.lambda_dssim
        for p, row in zip(res.plans, s.tolist()):
            npx = 3.0 * p.H * p.W
            total += (1 - lam) * row[0] / npx + lam * (1.0 - row[1] / npx)
        return total

    def _densify_and_reset(self, iteration: int, bs: int):
        o, a = self.opt, self.args
        if iteration >= o.densify_until_iter:
            return False
        changed = False
        if iteration >= o.densify_from_iter and is_interval_in_batch(iteration, bs, o.densification_interval):
            size_thr = 20 if iteration > o.opacity_reset_interval else None
            t0 = time.time()
            for m, st in self.stores.items():
                info = densify.densify_and_prune(st, o.densify_grad_threshold, 0.005, self.cameras_extent, size_thr,
                                                 o.percent_dense, a.MAX_SIZE_SINGLE_GS, False, a.SKIP_CLONE, a.SKIP_SPLIT,
                                                 self._gen)
                self.logger.info("model %d -> %d points at iteration %d (%s)", m, st.count, iteration, info)
                if self.tb:
                    self.tb.add_scalar(f"total_points_{m}", st.count, iteration)
            if self.tb:
                self.tb.add_scalar("cnt/densify_and_prune", time.time() - t0, iteration)
            changed = True
        if is_interval_in_batch(iteration, bs, o.opacity_reset_interval) or \
                (self.mdp.white_background and is_point_in_batch(iteration, bs, o.densify_from_iter)):
            for st in self.stores.values():
                densify.reset_opacity(st)
            if self.border is not None:
                self.border.invalidate()  # every opacity changed: the lent copies are stale
        if changed:
            self._spatial_sort()  # children were appended at the end: restore the memory locality of the rows
            for st in self.stores.values():
                st.zero_grad()  # rows moved: gradients of this step are dropped, like the reference's rebuilt optimiser
            if self.border is not None:
                self.border.invalidate()
        return changed

    # ------------------------------------------------------------------------------------------------
    # checkpoints
    # ------------------------------------------------------------------------------------------------
    def save(self, iteration: int) -> str:
        out = os.path.join(self.model_path, "point_cloud", f"iteration_{iteration}")
        os.makedirs(out, exist_ok=True)
        self.cleaner.add(out)
        lrs = self.learning_rates(iteration)
        for m, st in self.stores.items():
            ply_io.save_gaussians(os.path.join(out, f"point_cloud_{m}.ply"), st.views(), self.sh_degree)
            torch.save(st.optimizer_state_dict(lrs), os.path.join(out, f"adam_{m}.pt"))
        if self.rank == 0:
            self.tree.save(os.path.join(out, "tree_0.txt"))
        self.logger.info("saved iteration %d to %s", iteration, out)
        return out

    def save_whole_model(self, iteration: int):
        """Merge every rank's sub-model files into one vanilla-3DGS ``point_cloud.ply`` (rank 0;
        ``scene/gaussian_nn_module.py:58-132``). The files are concatenated block by block, never loaded."""
        files = sorted(glob.glob(os.path.join(self.model_root, "rank_*", "point_cloud", f"iteration_{iteration}", "point_cloud_*.ply")))
        if not files:
            return
        out = os.path.join(self.model_root, "point_cloud", f"iteration_{iteration}")
        os.makedirs(out, exist_ok=True)
        n = ply_io.merge_gaussian_files(os.path.join(out, "point_cloud.ply"), files, self.sh_degree)
        self.logger.info("merged %d sub-model files (%d Gaussians) into %s", len(files), n, out)

    # ------------------------------------------------------------------------------------------------
    # evaluation
    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def eval(self) -> dict:
        a = self.args
        results = {}
        sh_deg = min(self.sh_degree, self.iteration // 1000) if self.load_iteration <= 0 or not a.EVAL_ONLY else self.sh_degree
        if a.EVAL_ONLY:
            sh_deg = self.sh_degree
        n_tr = len(self.train_dataset)
        splits = (("train", DatasetRepeater(self.train_dataset, n_tr // max(a.EVAL_PSNR_INTERVAL, 1), False, a.EVAL_PSNR_INTERVAL),
                   self.train_rlt, a.EVAL_PSNR_INTERVAL), ("test", self.test_dataset, self.test_rlt, 1))
        if not hasattr(self, "_lpips"):
            from .utils.lpips import load_lpips
            self._lpips = load_lpips(getattr(a, "LPIPS_WEIGHTS", ""), self.device)
        self.eval_stamps = []
        for name, ds, rlt, stride in splits:
            stat = torch.zeros(4, dtype=torch.float64, device=self.device)  # samples, l1, psnr, ssim
            lp_sum, lp_n = 0.0, 0
            step = max(a.MAX_BATCH_SIZE, 1)
            feed = BatchPrefetcher(ds, [range(b0, min(len(ds), b0 + step)) for b0 in range(0, len(ds), step)],
                                   depth=self._prefetch_depth(), workers=getattr(a, "PREFETCH_WORKERS", 8))
            for idx, cams in feed:  # the targets of the next batches are decoded while this one is rendered
                idx = list(idx)
                rel = rlt[[(i * stride) % max(len(rlt), 1) for i in idx]]
                outs = self.engine.render(cams, rel, sh_deg, self.background)
                for cam, out in zip(cams, outs):
                    cl = self.engine._loss(out["plan"].view, cam.height, cam.width)
                    r0, r1 = out["rows"]
                    gt = self.engine._gt_rows(out["plan"].view, cam, (max(0, r0 - 5), min(cam.height, r1 + 5)))
                    # SSIM needs the composited neighbours: composite the halo rows as well
                    sums = torch.zeros(6, dtype=torch.float64, device=self.device)
                    if r1 > r0:
                        sums[:3] = cl.stats(gt, r0, r1)
                        # squared error per colour channel: the reference's PSNR is the mean over the channels of the
                        # per-channel PSNR (utils/image_utils.py:17-19), not the PSNR of the pooled error
                        sums[3:] = ((out["image"][:, r0:r1] - gt[:, r0:r1]).double() ** 2).sum(dim=(1, 2))
                    if self.world > 1:
                        dist.all_reduce(sums, group=self.group)
                    npx = 3.0 * cam.height * cam.width
                    l1, ssim, _ = (sums[:3] / npx).tolist()
                    psnr = sum(psnr_from_mse(v) for v in (sums[3:] / (npx / 3.0)).tolist()) / 3.0
                    stat += torch.tensor([1.0, l1, psnr, ssim], dtype=torch.float64, device=self.device)
                    self.eval_stamps.append((name, time.perf_counter()))  # the metrics were read back: the image is done
                    self.logger.info("%s, image %s, psnr %f, ssim %f, l1 %f", name, cam.image_name, psnr, ssim, l1)
                    if self.tb and cam.uid < 1000 and cam.uid % 5 == 0:
                        # every fifth view, render and ground truth (trainer4tree_partition.py:731-733 of the reference)
                        self._tb_images(name, cam, out, gt)
                    if self._lpips is not None:
                        # the perceptual metric needs whole images: the row bands are summed into one on every rank
                        full = torch.zeros(3, cam.height, cam.width, device=self.device)
                        full[:, r0:r1] = out["image"][:, r0:r1]
                        gt_full = torch.zeros_like(full)
                        gt_full[:, r0:r1] = gt[:, r0:r1]
                        if self.world > 1:
                            dist.all_reduce(full, group=self.group)
                            dist.all_reduce(gt_full, group=self.group)
                        lp_sum += float(self._lpips(full.clamp(0, 1), gt_full))
                        lp_n += 1
                    if a.SAVE_EVAL_IMAGE:
                        self._save_rows(out, cam, name)
                    if a.SAVE_EVAL_SUB_IMAGE:
                        for m, part in out["partials"].items():
                            save_png(os.path.join(self.model_root, "img", f"{name}_{cam.image_name}_{self.iteration}_sub_{m}.png"),
                                     part[..., :3].permute(2, 0, 1))
            n, l1, ps, ss = stat.tolist()
            n = max(n, 1.0)
            lp = lp_sum / lp_n if lp_n else float("nan")
            results[name] = dict(samples=n, l1=l1 / n, psnr=ps / n, ssim=ss / n, lpips=lp)
            if self.rank == 0:
                msg = f"\n[ITER {self.iteration}] Evaluating {name}: samples {n} L1 {l1 / n} PSNR {ps / n} SSIM {ss / n} LPIPS {lp}"
                print(msg, flush=True)
                self.logger.info(msg)
                if self.tb:
                    self.tb.add_scalar(name + "/loss_viewpoint - l1_loss", l1 / n, self.iteration)
                    self.tb.add_scalar(name + "/loss_viewpoint - psnr", ps / n, self.iteration)
                    self.tb.add_scalar(name + "/loss_viewpoint - ssim", ss / n, self.iteration)
                    self.tb.add_scalar(name + "/loss_viewpoint - lpips", lp, self.iteration)
        if self.tb:
            for m, st in self.stores.items():
                self.tb.add_scalar(f"total_points_{m}", st.count, self.iteration)
        return results

    def _tb_images(self, split: str, cam: Camera, out, gt: torch.Tensor):
        """Whole render and ground truth of one view to TensorBoard (the row bands are summed over the ranks)."""
        r0, r1 = out["rows"]
        full = torch.zeros(3, cam.height, cam.width, device=self.device)
        full[:, r0:r1] = out["image"][:, r0:r1]
        gt_full = torch.zeros_like(full)
        gt_full[:, r0:r1] = gt[:, r0:r1]
        if self.world > 1:
            dist.all_reduce(full, group=self.group)
            dist.all_reduce(gt_full, group=self.group)
        self.tb.add_images(f"{split}_view_{cam.image_name}/render", full.clamp(0, 1)[None].cpu(), global_step=self.iteration)
        self.tb.add_images(f"{split}_view_{cam.image_name}/ground_truth", gt_full[None].cpu(), global_step=self.iteration)

    def _save_rows(self, out, cam: Camera, split: str):
        """Gather the row bands of a composited image on rank 0 and write it (plus the ground truth)."""
        img = out["image"].clone()
        r0, r1 = out["rows"]
        full = torch.zeros_like(img)
        full[:, r0:r1] = img[:, r0:r1]
        if self.world > 1:
            dist.all_reduce(full, group=self.group)
        if self.rank == 0:
            save_png(os.path.join(self.model_root, "img", f"{split}_{cam.image_name}_{self.iteration}.png"), full)
            if cam.image is not None:
                save_png(os.path.join(self.model_root, "gt", f"{cam.image_name}.png"), cam.image)

    # ------------------------------------------------------------------------------------------------
    # repartition
    # ------------------------------------------------------------------------------------------------
    def _repartition(self):
        """Rebalance: all-reduce the load histogram, rebuild the tree away from the old split planes, move
        every Gaussian (parameters + Adam moments, 177 floats) to the sub-model whose box now holds its
        centre (``trainer4tree_partition.py:220-317``)."""
        self.logger.info("repartition at iteration %d: %s", self.iteration, {m: s.count for m, s in self.stores.items()})
        grid = self.tree.grid
        hist = torch.zeros(grid.grid_size, dtype=torch.float32, device=self.device)
        for st in self.stores.values():
            if st.count:
                hist += load_histogram(st.xyz, grid)
        if self.world > 1:
            dist.all_reduce(hist, group=self.group)
        grid.load = hist.double().cpu().numpy()
        new_tree = BvhTree.build(grid, self.bvh_depth, self.SPLIT_ORDERS, previous=self.tree,
                                 rng=np.random.default_rng(self.iteration)) if self.rank == 0 else None
        self.tree = self._bcast(new_tree)
        old = self.stores
        lo, hi = self._stores_from_tree()
        from .parallel.migrate import migrate
        self.stores = migrate(old, self.tree, lo, hi, self.model2rank, self.rank, self.world, self.device, self.sh_degree,
                              self.group)
        self._spatial_sort()
        for st in self.stores.values():
            st.active_sh_degree = min(self.sh_degree, self.iteration // 1000)
        self._close_engine()  # the old exchange regions are unmapped before new ones are created
        self._build_engine()
        self.train_rlt = self._relation(self.train_dataset, "trainset_relation.pt", use_cache=False)
        self.test_rlt = self._relation(self.test_dataset, "testset_relation.pt", use_cache=False)
