"""Benchmark session: the flagship training step on a seeded synthetic scene.

Builds, on every rank, the part of the scene that the rank hosts (cluster-mixture Gaussians cut by
the kd/BVH partition into one sub-model per GPU), renders ground-truth images from an independent
seeded scene into pinned host memory, and exposes ``step`` (device-timed loop) and ``step_e2e``
(host-timed loop that also reads the loss back).  The work per step is exactly the trainer's
``StepEngine.train_step``: ground-truth upload, render of every visible local sub-model, compositing,
L1 + D-SSIM loss, backward, fused Adam on every sub-model.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.distributed as dist

from .data import synthetic
from .engine import StepEngine
from .models.gaussians import GaussianStore
from .ops import native
from .ops.rasterize import RenderTask, Segment, make_camera
from .parallel.compositing import LocalTransport, TorchDistTransport
from .parallel.partition import BvhTree, Grid3D, assign_models, load_histogram

CHUNK = 4_000_000


class ClusterScene:
    """Seeded mixture of anisotropic 3D clusters, sampled in chunks so that no rank ever holds more than
    one chunk besides its own sub-models."""

    def __init__(self, seed: int, device, n_clusters: int = 64, box: float = 20.0):
        self.seed, self.device, self.box = seed, device, box
        g = torch.Generator(device=device)
        g.manual_seed(seed + 101)
        self.centers = (torch.rand(n_clusters, 3, device=device, generator=g) - 0.5) * box * 0.8
        self.centers[:, 2] = self.centers[:, 2].abs() * 0.5
        self.axes = 0.3 + 1.7 * torch.rand(n_clusters, 3, device=device, generator=g)
        # random rotations from normalised quaternions (element-wise arithmetic only: no solver library is involved)
        q = torch.nn.functional.normalize(torch.randn(n_clusters, 4, device=device, generator=g), dim=1)
        w, x, y, z = q.unbind(1)
        self.rot = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y),
                                2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x),
                                2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], dim=1).view(n_clusters, 3, 3)

    def means(self, n: int, chunk: int) -> torch.Tensor:
        g = torch.Generator(device=self.device)
        g.manual_seed(self.seed * 7919 + 13 * chunk + 1)
        which = torch.randint(0, self.centers.shape[0], (n,), device=self.device, generator=g)
        local = torch.randn(n, 3, device=self.device, generator=g) * self.axes[which]
        pts = torch.einsum("nij,nj->ni", self.rot[which], local) + self.centers[which]
        return pts.clamp_(-self.box / 2, self.box / 2)

    def gaussians(self, n: int, chunk: int, sh_degree: int = 3) -> dict:
        return synthetic.random_gaussians(n, self.means(n, chunk), self.seed * 104729 + chunk, self.device, sh_degree)


def chunks_of(n: int):
    k = 0
    while n > 0:
        m = min(n, CHUNK)
        yield k, m
        n -= m
        k += 1


class UniformScene:
    """Gaussians uniform in [-1,1]^3 with the plumbing-test statistics (log-scale N(-4,.5), SH degree 1)."""

    box = 2.0

    def __init__(self, seed: int, device):
        self.seed, self.device = seed, device

    def means(self, n: int, chunk: int) -> torch.Tensor:
        g = torch.Generator(device=self.device)
        g.manual_seed(self.seed * 7919 + 13 * chunk + 1)
        return torch.rand(n, 3, device=self.device, generator=g) * 2 - 1

    def gaussians(self, n: int, chunk: int, sh_degree: int = 1) -> dict:
        return synthetic.random_gaussians(n, self.means(n, chunk), self.seed * 104729 + chunk, self.device, sh_degree)


class AerialScene:
    """City-scale aerial scene in chunks: half of the Gaussians on a ground plane of ``box`` x ``box`` units (heights
    exponentially distributed), half in seeded building-like vertical boxes; log-scales around exp(-1) unit."""

    box = 2000.0
    kind = "aerial"

    def __init__(self, seed: int, device, n_buildings: int = 4096):
        self.seed, self.device = seed, device
        g = torch.Generator(device=device)
        g.manual_seed(seed + 211)
        self.bc = (torch.rand(n_buildings, 2, device=device, generator=g) - 0.5) * self.box
        self.bh = 10.0 + 60.0 * torch.rand(n_buildings, device=device, generator=g)
        self.bw = 5.0 + 20.0 * torch.rand(n_buildings, 2, device=device, generator=g)

    def means(self, n: int, chunk: int) -> torch.Tensor:
        g = torch.Generator(device=self.device)
        g.manual_seed(self.seed * 7919 + 13 * chunk + 1)
        dev = self.device
        n_ground = n // 2
        pts = torch.empty(n, 3, device=dev)
        pts[:n_ground, :2] = (torch.rand(n_ground, 2, device=dev, generator=g) - 0.5) * self.box
        pts[:n_ground, 2] = -3.0 * torch.log(torch.rand(n_ground, device=dev, generator=g).clamp_min(1e-6))
        nb = n - n_ground
        which = torch.randint(0, self.bc.shape[0], (nb,), device=dev, generator=g)
        pts[n_ground:, :2] = self.bc[which] + (torch.rand(nb, 2, device=dev, generator=g) - 0.5) * self.bw[which]
        pts[n_ground:, 2] = torch.rand(nb, device=dev, generator=g) * self.bh[which]
        half = self.box / 2
        pts[:, :2].clamp_(-half, half)
        return pts

    def gaussians(self, n: int, chunk: int, sh_degree: int = 3) -> dict:
        return synthetic.random_gaussians(n, self.means(n, chunk), self.seed * 104729 + chunk, self.device, sh_degree,
                                          log_scale_mean=-1.0)


class BenchSession:
    def __init__(self, device, rank: int, world: int, n_gaussians: int, width: int, height: int, batch: int,
                 n_views: int, gt_gaussians: int, transport: str = "auto", seed: int = 0, sh_degree: int = 3,
                 grid=(2048, 2048, 1), bvh_depth: int | None = None, scene_kind: str = "cluster",
                 borrow: bool = True, borrow_refresh: int = 1, group=None, spatial_sort: bool = True,
                 pool_views: int = 0, balance_batches: bool = False):
        self.device = torch.device(device)
        self.rank, self.world, self.batch = rank, world, batch
        self.sh_degree = sh_degree
        self.bvh_depth = int(round(math.log2(world))) if bvh_depth is None else bvh_depth
        assert 2 ** self.bvh_depth >= world, "need at least one sub-model per rank"
        make_scene = {"cluster": ClusterScene, "aerial": AerialScene}.get(scene_kind, UniformScene)
        self._make_scene = make_scene
        scene = make_scene(seed, self.device)
        # ---- partition from the load histogram of all positions -------------------------------
        half = scene.box / 2
        g3 = Grid3D(np.array([-half] * 3), np.array([half] * 3), grid)
        hist = torch.zeros(grid, dtype=torch.float32, device=self.device)
        for k, m in chunks_of(n_gaussians):
            hist += load_histogram(scene.means(m, k), g3)
        g3.load = hist.double().cpu().numpy()
        self.tree = BvhTree.build(g3, self.bvh_depth, (0, 1))
        self.n_models = len(self.tree.leaves)
        self.model2rank = assign_models(self.n_models, world)
        lo, hi = self.tree.leaf_boxes_world(open_border=True)
        local = [m for m in range(self.n_models) if self.model2rank[m] == rank]
        counts = {m: 0 for m in local}
        # ---- fill the local sub-models chunk by chunk -------------------------------------------
        self.stores = {m: GaussianStore(max(4, int(n_gaussians / self.n_models * 1.15)), self.device, sh_degree,
                                        lo[m], hi[m], m) for m in local}
        for st in self.stores.values():
            st.active_sh_degree = sh_degree
        for k, mcount in chunks_of(n_gaussians):
            g = scene.gaussians(mcount, k, sh_degree)
            ids = self.tree.label(g["xyz"])
            for m in local:
                sel = (ids == m).nonzero(as_tuple=True)[0]
                if sel.numel():
                    self.stores[m].append_new({name: v[sel] for name, v in g.items()})
            del g, ids
        if spatial_sort:  # rows along a space-filling curve: the visible rows of a view lie close together in memory
            for st in self.stores.values():
                st.spatial_sort()
        torch.cuda.empty_cache() if self.device.type == "cuda" else None
        # ---- cameras, relation, ground truth -----------------------------------------------------
        if scene_kind == "cluster":
            self.cams = synthetic.hemisphere_cameras(max(n_views, 1), 8.0, width, height, 50.0, seed)
        elif scene_kind == "aerial":
            self.cams = synthetic.aerial_cameras(max(n_views, 1), scene.box, width, height, 60.0, seed)
        else:
            self.cams = synthetic.ring_cameras(max(n_views, 1), 3.0, width, height, 60.0)
        self.relation = self.tree.relation(self.cams, 0.01, 1000.0)
        self.batches = None
        if pool_views > len(self.cams) and scene_kind == "cluster":
            self._batches_from_pool(pool_views, n_views, width, height, seed, balance_batches, group)
        self._render_ground_truth(seed, gt_gaussians, sh_degree)
        # ---- engine ---------------------------------------------------------------------------
        self.transport_name = "local"
        tr = LocalTransport(self.device)
        if world > 1:
            want = transport
            if want in ("auto", "peer"):
                try:
                    from .parallel.peer import PeerTransport
                    tr = PeerTransport(self.device, group)
                    self.transport_name = "peer (kernel stores into peer-mapped slots, flag barrier)"
                except Exception as exc:  # pragma: no cover - depends on the box
                    if want == "peer":
                        raise
                    if rank == 0:
                        print(f"[bench] peer transport unavailable ({exc!r}); using torch.distributed send/recv",
                              flush=True)
                    tr = TorchDistTransport(self.device, group)
                    self.transport_name = "torch.distributed send/recv"
            else:
                tr = TorchDistTransport(self.device, group)
                self.transport_name = "torch.distributed send/recv"
        self.border = None
        if borrow and self.n_models > 1:
            from .parallel.border import BorderExchange
            if hasattr(tr, "push_plan"):  # peer transport: border rows travel by peer stores as well
                from .parallel.peer_border import PeerBorderExchange
                self.border = PeerBorderExchange(lo, hi, self.model2rank, rank, world, self.device, tr, group, borrow_refresh)
            else:
                self.border = BorderExchange(lo, hi, self.model2rank, rank, world, self.device, group, borrow_refresh)
        self.borrow_refresh = borrow_refresh
        self.engine = StepEngine(self.stores, self.model2rank, self.device, tr, borrow=self.border)
        extent = 1.1 * 8.0 if scene_kind != "aerial" else 1.1 * 0.5 * scene.box
        self.extent = extent
        self.group = group
        self.lrs = (1.6e-4 * extent, 2.5e-3, 2.5e-3 / 20.0, 5e-3, 1e-3, 5e-2)
        self.last_info: dict = {}
        self._launch_base = 0

    def _batches_from_pool(self, pool_views: int, n_views: int, width: int, height: int, seed: int, balance: bool, group):
        """Batches as the trainer forms them: a seeded shuffle of a pool of training cameras packed into batches, either
        in sequence (the reference's balancer, ``utils/workload_utils.py:20-59``) or, with ``balance``, pairing cameras
        whose estimated per-rank loads complement each other (``WorkloadBalancer.groups_balanced``, the trainer's
        ``--BALANCE_BATCHES``). Only the cameras of the first ``n_views / batch`` batches are kept (and get targets)."""
        from .parallel.balancer import WorkloadBalancer, estimate_costs
        pool = synthetic.hemisphere_cameras(pool_views, 8.0, width, height, 50.0, seed)
        rel = self.tree.relation(pool, 0.01, 1000.0)
        g = torch.Generator()
        g.manual_seed(seed)
        order = torch.randperm(pool_views, generator=g).tolist()
        bal = WorkloadBalancer(self.world, self.model2rank)
        max_task = self.batch * max(2, -(-self.n_models // self.world))
        if balance and self.world > 1:
            cost = torch.from_numpy(estimate_costs(self.stores, pool, self.n_models)).to(self.device)
            dist.all_reduce(cost, group=group)
            groups = bal.groups_balanced(rel, order, cost.cpu().numpy(), max_task, self.batch)
        else:
            groups = bal.groups(rel, order, max_task, self.batch)
        groups = [g_ for g_ in groups if len(g_) == self.batch][:max(1, n_views // self.batch)]
        used = [i for g_ in groups for i in g_]
        remap = {i: k for k, i in enumerate(used)}
        self.cams = [pool[i] for i in used]
        for k, cam in enumerate(self.cams):
            cam.uid = k
        self.relation = rel[used]
        self.batches = [tuple(remap[i] for i in g_) for g_ in groups]

    # -- ground truth -----------------------------------------------------------------------------
    def _render_ground_truth(self, seed: int, gt_gaussians: int, sh_degree: int):
        """Targets come from an independent seeded scene; each view is rendered once and parked in pinned
        host memory (only the rows this rank owns, plus the SSIM halo, are uploaded per step)."""
        scene = self._make_scene(seed + 1, self.device)
        parts = [scene.gaussians(m, k, sh_degree) for k, m in chunks_of(gt_gaussians)]
        g = {name: torch.cat([p[name] for p in parts]) for name in parts[0]}
        seg = Segment(g["xyz"], g["sh"], g["scale"], g["rot"], g["opacity"])
        task = RenderTask(self.device)
        pin = self.device.type == "cuda"
        for cam in self.cams:
            c = make_camera(cam, sh_degree)
            out = task.forward(c, [seg], check=True)
            img = out[..., :3].permute(2, 0, 1).contiguous().cpu()
            cam.image = img.pin_memory() if pin else img
        del task, seg, g, parts
        from .ops import rasterize
        rasterize.release_scratch()
        if pin:
            torch.cuda.empty_cache()

    # -- steps ------------------------------------------------------------------------------------
    def _batch(self, i: int):
        if self.batches:
            idx = list(self.batches[i % len(self.batches)])
        else:
            idx = [(i * self.batch + j) % len(self.cams) for j in range(self.batch)]
        return [self.cams[k] for k in idx], self.relation[idx]

    def step(self, i: int):
        cams, rel = self._batch(i)
        return self.engine.train_step(cams, rel, self.sh_degree, self.lrs)

    def step_e2e(self, i: int):
        cams, rel = self._batch(i)
        res = self.engine.train_step(cams, rel, self.sh_degree, self.lrs)
        sums = torch.stack(res.sums).cpu()  # device -> host read of the step's loss sums
        loss = 0.0
        for p, s in zip(res.plans, sums):
            npx = 3.0 * p.H * p.W
            b = p.bands[self.rank]
            # this rank's share of (1-lambda) L1 + lambda (1 - SSIM); shares of all ranks add up to the loss
            loss += (0.8 * float(s[0]) + 0.2 * (3.0 * (b[1] - b[0]) * p.W - float(s[1]))) / npx
        h2d = 0
        for p in res.plans:
            b = p.bands[self.rank]
            if b[1] > b[0]:
                h2d += 3 * (min(p.H, b[1] + 5) - max(0, b[0] - 5)) * p.W * 4
        return loss, h2d, int(sums.numel() * 8)

    # -- model surgery at scale (what the trainer does every densification interval / repartition epoch) ------------
    def densify(self, grad_threshold: float = 2e-4) -> dict:
        """Clone / split / prune every local sub-model from the statistics gathered by the steps so far."""
        from .models import densify as dz
        info = {}
        for m, st in self.stores.items():
            info[m] = dz.densify_and_prune(st, grad_threshold, 0.005, self.extent, None, 0.01, None, False, False, False,
                                           None, seed=1234 + m)
            st.zero_grad()
        if self.border is not None:
            self.border.invalidate()
        return info

    def repartition(self) -> dict:
        """Rebuild the kd-tree from the current load and move every Gaussian (parameters + Adam moments) to the sub-model
        whose new box holds it; returns counts and the engine is rebuilt on the new stores."""
        from .parallel.migrate import migrate
        grid = self.tree.grid
        hist = torch.zeros(grid.grid_size, dtype=torch.float32, device=self.device)
        for st in self.stores.values():
            if st.count:
                hist += load_histogram(st.xyz, grid)
        if self.world > 1:
            dist.all_reduce(hist, group=self.group)
        grid.load = hist.double().cpu().numpy()
        new_tree = BvhTree.build(grid, self.bvh_depth, (0, 1), previous=self.tree, rng=np.random.default_rng(7))
        lo, hi = new_tree.leaf_boxes_world(open_border=True)
        moved = sum(int((new_tree.label(st.xyz) != m).sum()) for m, st in self.stores.items() if st.count)
        before = sum(st.count for st in self.stores.values())
        if self.border is not None and hasattr(self.border, "close"):
            self.border.close()
        if hasattr(self.engine.transport, "close"):
            self.engine.transport.close()
        self.stores = migrate(self.stores, new_tree, lo, hi, self.model2rank, self.rank, self.world, self.device,
                              self.sh_degree, self.group)
        self.tree = new_tree
        for st in self.stores.values():
            st.active_sh_degree = self.sh_degree
            st.spatial_sort()
        self.relation = self.tree.relation(self.cams, 0.01, 1000.0)
        tr = self.engine.transport.__class__(self.device, self.group) if self.world > 1 else LocalTransport(self.device)
        self.border = None
        if self.n_models > 1 and self.engine.borrow is not None:
            if hasattr(tr, "push_plan"):
                from .parallel.peer_border import PeerBorderExchange
                self.border = PeerBorderExchange(lo, hi, self.model2rank, self.rank, self.world, self.device, tr, self.group,
                                                 self.borrow_refresh)
            else:
                from .parallel.border import BorderExchange
                self.border = BorderExchange(lo, hi, self.model2rank, self.rank, self.world, self.device, self.group,
                                             self.borrow_refresh)
        self.engine = StepEngine(self.stores, self.model2rank, self.device, tr, borrow=self.border)
        return dict(moved=moved, before=before, after=sum(st.count for st in self.stores.values()))

    def settle(self) -> bool:
        """Synchronise and let every render task look at its counters (grows buffers after an overflow)."""
        self.sync()
        info = self.engine.poll()
        self.last_info = info
        return bool(info["overflow"])

    def sync(self):
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def barrier(self):
        if self.world > 1:
            dist.barrier()

    def render_view(self, i: int):
        """Composited image rows owned by this rank for camera ``i`` (eval path)."""
        out = self.engine.render([self.cams[i]], self.relation[[i]], self.sh_degree)[0]
        return out["image"], out["rows"], out["trans"]

    def reset_launch_count(self):
        self._launch_base = native.launch_count()

    def launch_count(self) -> int:
        return native.launch_count() - self._launch_base


def phase_roofline(phases: dict, views_per_step: int, n_gaussians: int, n_vis: int, n_inst: int, live_rows: int, height: int,
                   width: int, partials: int, hbm_gbs: float | None) -> dict:
    """Algorithmic bytes per step of the memory-bound phases and what they make of the measured phase times.

    ``phases``: ms per step and phase (``PhaseTimer.table``); ``n_vis`` / ``n_inst``: visible splats and tile instances
    of one step on this rank; ``live_rows``: rows the Adam kernel updates; ``partials``: partial images per view. The
    byte counts are what the kernels must move at least (each operand once): cull 24 B per Gaussian and view, projection
    236 B in + 110 B out per visible splat, depth sort 4 passes and tile sort 2 passes of 8-byte pairs (read + write +
    4 B histogram read), emission 8 B per instance, compositing + loss ~32 B per pixel and partial + 160 B per pixel,
    Adam 1416 B per live row + 2 mark bytes per row. The blend kernels are instruction-bound and have no entry.
    Fractions are of the measured copy bandwidth (``hbm_gbs``) when it is known.
    """
    model = {
        "fwd.project": views_per_step * 24.0 * n_gaussians + 346.0 * n_vis,
        "fwd.binning": 104.0 * n_vis + 48.0 * n_inst,
        "composite_loss": views_per_step * float(height) * width * (32.0 * partials + 160.0),
        "adam": 1416.0 * live_rows + 2.0 * n_gaussians,
    }
    out = {}
    for name, nbytes in model.items():
        ms = phases.get(name)
        if not ms:
            continue
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 3), "algorithmic_gb": round(nbytes / 1e9, 3), "gb_per_s": round(gbs, 1),
                     "frac_of_measured_hbm": round(gbs / hbm_gbs, 3) if hbm_gbs else None}
    return out
