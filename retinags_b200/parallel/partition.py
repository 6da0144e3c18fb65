"""Spatial partition: load grid, kd/BVH tree of sub-model boxes, camera -> sub-model relation.

Behavioural parity with the reference's ``parallel_utils/grid_utils/utils.py`` (grid ``:154-180``,
median-of-load split with margin and jitter ``:228-263``, BFS build ``:334-360``, pickle layout
``:363-382``, rebuild from file ``:385-402``) and ``basic_parallel_trainer/scene_utils.py``
(leaf order and model->rank map ``:185-218``, relation vector ``:220-264``).  Differences:

* pure NumPy; the grid does not need a GPU (the reference's ``Grid3DSpace`` allocates CUDA tensors);
  the load histogram of resident Gaussians is computed on their device (``load_histogram``).
* box/frustum overlap is an exact separating-axis test, vectorised over all (camera, leaf) pairs,
  instead of one ``scipy.spatial.ConvexHull`` of a Minkowski difference per pair (``:115-137``).
* leaves that touch the border of the grid extend to infinity on that side when used as clip boxes,
  so Gaussians that drift out of the initial bounding box are still rendered by someone.
"""
from __future__ import annotations

import pickle
from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class Grid3D:
    range_low: np.ndarray
    range_up: np.ndarray
    grid_size: tuple
    load: np.ndarray = field(default=None, repr=False)

    def __post_init__(self):
        self.range_low = np.asarray(self.range_low, dtype=np.float64)
        self.range_up = np.asarray(self.range_up, dtype=np.float64)
        self.grid_size = tuple(int(v) for v in self.grid_size)
        self.voxel_size = (self.range_up - self.range_low) / np.asarray(self.grid_size, dtype=np.float64)
        self.voxel_size = np.maximum(self.voxel_size, 1e-12)
        if self.load is None:
            self.load = np.zeros(self.grid_size, dtype=np.float64)

    @classmethod
    def from_points(cls, pts: np.ndarray, grid_size) -> "Grid3D":
        lo, hi = pts.min(axis=0), pts.max(axis=0)
        return cls(lo, hi, grid_size)

    def cell_index(self, pos: np.ndarray) -> np.ndarray:
        idx = np.floor((pos - self.range_low) / self.voxel_size).astype(np.int64)
        return np.clip(idx, 0, np.asarray(self.grid_size) - 1)

    def clear(self):
        self.load[...] = 0

    def accumulate(self, pos: np.ndarray, load: np.ndarray | None = None):
        idx = self.cell_index(np.asarray(pos, dtype=np.float64))
        flat = np.ravel_multi_index((idx[:, 0], idx[:, 1], idx[:, 2]), self.grid_size)
        w = None if load is None else np.asarray(load, dtype=np.float64)
        self.load += np.bincount(flat, weights=w, minlength=int(np.prod(self.grid_size))).reshape(self.grid_size)

    def to_world(self, cell) -> np.ndarray:
        return np.asarray(cell, dtype=np.float64) * self.voxel_size + self.range_low


def load_histogram(xyz: torch.Tensor, grid: Grid3D, weights: torch.Tensor | None = None) -> torch.Tensor:
    """Per-cell load of Gaussians resident on ``xyz.device`` (replaces the reference's CPU numba
    scatter-add ``accum_on_3Dgrid``, ``grid_utils/utils.py:140-151``).  Returns a float32 tensor of the grid's shape on
    the same device, ready to be all-reduced.  Native kernel: ``rgs_histogram_kernel`` (``csrc/rgs_aux.cu``)."""
    import ctypes

    from ..ops import native
    out = torch.zeros(grid.grid_size, dtype=torch.float32, device=xyz.device)
    n = int(xyz.shape[0])
    if n == 0:
        return out
    lo = (ctypes.c_double * 3)(*[float(v) for v in grid.range_low])
    vs = (ctypes.c_double * 3)(*[float(v) for v in grid.voxel_size])
    dims = (ctypes.c_int64 * 3)(*[int(v) for v in grid.grid_size])
    w = None if weights is None else weights.detach().float().contiguous()
    native.call("histogram", xyz.device, xyz.detach().float().contiguous(), w, n, lo, vs, dims, out, sig="ppippppp")
    return out


@dataclass
class BvhNode:
    range_low: tuple
    range_up: tuple
    level: int
    path: str
    split_orders: list
    split_position: int | None = None
    left: "BvhNode | None" = None
    right: "BvhNode | None" = None

    @property
    def split_dim(self) -> int:
        return self.split_orders[self.level % len(self.split_orders)]

    @property
    def is_leaf(self) -> bool:
        return self.left is None and self.right is None

    @property
    def size(self) -> int:
        return int(np.prod(np.asarray(self.range_up) - np.asarray(self.range_low)))


class BvhTree:
    """kd-tree over grid cells; leaves sorted by path are the sub-models 0..M-1."""

    def __init__(self, grid: Grid3D, nodes: dict[str, BvhNode]):
        self.grid = grid
        self.nodes = nodes
        self.leaves = sorted((n for n in nodes.values() if n.is_leaf), key=lambda n: n.path)

    # -- construction ---------------------------------------------------------------------------
    @classmethod
    def build(cls, grid: Grid3D, max_depth: int, split_orders=(0, 1), previous: "BvhTree | None" = None,
              rng: np.random.Generator | None = None) -> "BvhTree":
        rng = rng or np.random.default_rng(0)
        root = BvhNode((0, 0, 0), tuple(grid.grid_size), 0, "", list(split_orders))
        nodes, queue = {}, [root]
        while queue:
            node = queue.pop(0)
            if node.level < max_depth:
                old = previous.nodes[node.path].split_position if previous and node.path in previous.nodes else None
                for child in cls._split(grid, node, 2 ** (max_depth - node.level), old, rng):
                    queue.append(child)
            nodes[node.path] = node
        return cls(grid, nodes)

    @staticmethod
    def _split(grid: Grid3D, node: BvhNode, limit: int, invalid: int | None, rng, radius: int = 10):
        d = node.split_dim
        if node.range_up[d] - node.range_low[d] < 2:
            return []
        sl = tuple(slice(l, u) for l, u in zip(node.range_low, node.range_up))
        load = grid.load[sl].sum(axis=tuple(i for i in range(3) if i != d))
        cum = np.cumsum(load)
        split = int(np.argmin(np.abs(2 * cum - load.sum())))
        if invalid is not None and node.range_low[d] + split + 1 == invalid:
            off = 0
            while off == 0:
                off = int(rng.integers(-radius, radius + 1))
            split += off
        limit = int(np.clip(limit, 0, len(load) // 2))
        split = int(np.clip(split, limit, len(load) - 1 - limit))
        pos = node.range_low[d] + split + 1
        node.split_position = pos
        lup, rlow = list(node.range_up), list(node.range_low)
        lup[d] = pos
        rlow[d] = pos
        node.left = BvhNode(node.range_low, tuple(lup), node.level + 1, node.path + "0", node.split_orders)
        node.right = BvhNode(tuple(rlow), node.range_up, node.level + 1, node.path + "1", node.split_orders)
        return [node.left, node.right]

    # -- files (the reference's pickle layout) ---------------------------------------------------
    def save(self, file_path: str):
        d = {p: [tuple(n.range_low), tuple(n.range_up), list(n.split_orders)] for p, n in self.nodes.items()}
        d["grid_info"] = [self.grid.range_low.astype(np.float32), self.grid.range_up.astype(np.float32),
                          tuple(self.grid.grid_size)]
        with open(file_path, "wb") as f:
            pickle.dump(d, f)

    @classmethod
    def load(cls, file_path: str) -> "BvhTree":
        with open(file_path, "rb") as f:
            d = pickle.load(f)
        lo, hi, gs = d.pop("grid_info")
        grid = Grid3D(np.asarray(lo), np.asarray(hi), tuple(int(v) for v in gs))
        nodes = {p: BvhNode(tuple(int(v) for v in lo_), tuple(int(v) for v in up_), len(p), p, list(so))
                 for p, (lo_, up_, so) in d.items()}
        for p, n in nodes.items():
            if p + "0" in nodes and p + "1" in nodes:
                n.left, n.right = nodes[p + "0"], nodes[p + "1"]
                n.split_position = n.right.range_low[n.split_dim]
        return cls(grid, nodes)

    # -- geometry -------------------------------------------------------------------------------
    def split_world(self, node: BvhNode) -> float:
        d = node.split_dim
        return float(node.split_position * self.grid.voxel_size[d] + self.grid.range_low[d])

    def leaf_boxes_grid(self) -> np.ndarray:
        return np.asarray([list(n.range_low) + list(n.range_up) for n in self.leaves], dtype=np.int64)

    def leaf_boxes_world(self, open_border: bool = False) -> tuple[np.ndarray, np.ndarray]:
        """(M,3) lower and upper corners in world units; with ``open_border`` the sides that coincide
        with the grid border are +-inf (clip boxes)."""
        g = self.leaf_boxes_grid()
        lo, hi = self.grid.to_world(g[:, :3]), self.grid.to_world(g[:, 3:])
        if open_border:
            lo = np.where(g[:, :3] == 0, -np.inf, lo)
            hi = np.where(g[:, 3:] == np.asarray(self.grid.grid_size), np.inf, hi)
        return lo, hi

    def label(self, xyz: torch.Tensor) -> torch.Tensor:
        """Sub-model id of every position (lo < p <= hi along the split planes; outside -> nearest leaf)."""
        ids = torch.zeros(xyz.shape[0], dtype=torch.int64, device=xyz.device)
        paths = {n.path: i for i, n in enumerate(self.leaves)}

        def rec(node: BvhNode, mask: torch.Tensor):
            if node.is_leaf:
                ids[mask] = paths[node.path]
                return
            right = xyz[:, node.split_dim] > self.split_world(node)
            rec(node.left, mask & ~right)
            rec(node.right, mask & right)

        rec(self.nodes[""], torch.ones(xyz.shape[0], dtype=torch.bool, device=xyz.device))
        return ids

    # -- relation -------------------------------------------------------------------------------
    def order_for(self, center: np.ndarray) -> list[int]:
        """Front-to-back position of every leaf for a camera centre: at each internal node the child
        that contains the centre comes first."""
        keys = []
        for mid, leaf in enumerate(self.leaves):
            bits = []
            for k in range(len(leaf.path)):
                parent = self.nodes[leaf.path[:k]]
                in_right = center[parent.split_dim] > self.split_world(parent)
                near = "1" if in_right else "0"
                bits.append(0 if leaf.path[k] == near else 1)
            keys.append((tuple(bits), mid))
        keys.sort()
        order = [0] * len(self.leaves)
        for pos, (_, mid) in enumerate(keys):
            order[mid] = pos
        return order

    def relation(self, cameras, z_near: float = 0.01, z_far: float = 1000.0) -> np.ndarray:
        """(N_cam, M) int32: front-to-back index of each visible sub-model, -1 when its box misses the
        frustum; an all -1 row becomes all 0 (``scene_utils.py:313-316``)."""
        lo, hi = self.leaf_boxes_world()
        M = len(self.leaves)
        rel = np.full((len(cameras), M), -1, dtype=np.int32)
        for i, cam in enumerate(cameras):
            order = self.order_for(np.asarray(cam.camera_center, dtype=np.float64))
            vis = frustum_overlaps_boxes(cam, lo, hi, z_near, z_far)
            for m in range(M):
                if vis[m]:
                    rel[i, m] = order[m]
            if (rel[i] < 0).all():
                rel[i] = 0
        return rel


def frustum_corners(cam, z_near: float, z_far: float) -> np.ndarray:
    """(8,3) world-space corners of the view frustum."""
    tx, ty = cam.tan_fovx, cam.tan_fovy
    pts = []
    for z in (z_near, z_far):
        for sx, sy in ((-1, -1), (1, -1), (1, 1), (-1, 1)):
            pts.append([sx * tx * z, sy * ty * z, z, 1.0])
    c2w_t = np.asarray(cam.view_world_transform, dtype=np.float64)
    return (np.asarray(pts, dtype=np.float64) @ c2w_t)[:, :3]


def frustum_overlaps_boxes(cam, lo: np.ndarray, hi: np.ndarray, z_near: float, z_far: float) -> np.ndarray:
    """Exact convex overlap test (separating axes) between the frustum and M axis-aligned boxes."""
    fc = frustum_corners(cam, z_near, z_far)  # near 0-3, far 4-7
    box_axes = np.eye(3)
    e_side = [fc[4 + k] - fc[k] for k in range(4)]
    e_h, e_v = fc[1] - fc[0], fc[3] - fc[0]
    f_edges = e_side + [e_h, e_v]
    f_normals = [np.cross(e_h, e_v)] + [np.cross(e_side[k], fc[(k + 1) % 4] - fc[k]) for k in range(4)]
    axes = list(box_axes) + f_normals + [np.cross(a, b) for a in box_axes for b in f_edges]
    axes = np.asarray([a / np.linalg.norm(a) for a in axes if np.linalg.norm(a) > 1e-12])
    fproj = fc @ axes.T  # (8,A)
    fmin, fmax = fproj.min(0), fproj.max(0)
    M = lo.shape[0]
    corners = np.stack([np.where(np.asarray(mask)[None, :], hi, lo)
                        for mask in [(a, b, c) for a in (0, 1) for b in (0, 1) for c in (0, 1)]], axis=1)  # (M,8,3)
    bproj = corners @ axes.T  # (M,8,A)
    bmin, bmax = bproj.min(1), bproj.max(1)
    separated = (bmax < fmin[None]) | (bmin > fmax[None])
    return ~separated.any(axis=1)


def assign_models(num_models: int, world: int, costs=None) -> list[int]:
    """Sub-model -> rank map. Without costs sub-model i lives on rank i % world (``scene_utils.py:185-189``). With
    one cost per sub-model (and more sub-models than ranks) the costliest sub-model goes first to the rank that
    carries least so far; every rank holds at least one sub-model, and ties fall to the lower rank, so that all
    ranks compute the same map from the same costs."""
    if costs is None or num_models <= world:
        return [i % world for i in range(num_models)]
    costs = [float(c) for c in costs]
    if len(costs) != num_models:
        raise ValueError("one cost per sub-model")
    order = sorted(range(num_models), key=lambda m: (-costs[m], m))
    load, held, out = [0.0] * world, [0] * world, [0] * num_models
    for pos, m in enumerate(order):
        left = num_models - pos
        empty = [r for r in range(world) if held[r] == 0]
        pool = empty if len(empty) >= left else range(world)
        r = min(pool, key=lambda q: (load[q], q))
        out[m] = r
        load[r] += costs[m]
        held[r] += 1
    return out
