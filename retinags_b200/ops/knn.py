"""Mean squared distance to the three nearest neighbours (initial Gaussian scale).

Stands in for ``simple_knn._C.distCUDA2``, which the reference imports from a submodule it does not ship
(``scene/gaussian_nn_module.py:413-414``): ``scales = log(sqrt(clamp_min(dist2, 1e-7)))``.  The points are
sorted by the cell of a uniform grid sized for a few points per cell; the native kernel (``csrc/rgs_knn.h``,
``csrc/rgs_aux.cu``; CPU twin in ``csrc/rgs_cpu.cpp``) searches cells ring by ring around each query until
its third neighbour is provably nearest, so the result is exact.
"""
from __future__ import annotations

import ctypes

import torch

from . import native


class RgsKnnGrid(ctypes.Structure):
    _fields_ = [("lo", ctypes.c_float * 3), ("cell", ctypes.c_float), ("dims", ctypes.c_int * 3)]


def brute_force(points: torch.Tensor, chunk: int = 4096) -> torch.Tensor:
    """O(P^2) reference used by the tests."""
    out = torch.empty(points.shape[0], device=points.device)
    for s in range(0, points.shape[0], chunk):
        d = torch.cdist(points[s:s + chunk].double(), points.double()).pow(2).float()
        v = torch.topk(d, min(4, points.shape[0]), dim=1, largest=False).values[:, 1:]
        out[s:s + chunk] = v.mean(1) if v.shape[1] else 0.0
    return out


def knn3_dist2(points: torch.Tensor, per_cell: float = 4.0, max_cells: int = 1 << 26) -> torch.Tensor:
    """(P,3) float32 -> (P,) mean of the squared distances to the 3 nearest other points."""
    P = points.shape[0]
    dev = points.device
    if P == 0:
        return torch.zeros(0, device=dev)
    pts = points.detach().float().contiguous()
    lo, hi = pts.min(0).values, pts.max(0).values
    ext = torch.clamp(hi - lo, min=1e-6)
    cell = float((ext.prod().item() * per_cell / max(P, 1)) ** (1.0 / 3.0))
    cell = max(cell, float(ext.max().item()) / 1024.0, 1e-9)
    dims = torch.clamp((ext / cell).floor().long() + 1, min=1)
    while int(dims.prod().item()) > max_cells:
        cell *= 1.26
        dims = torch.clamp((ext / cell).floor().long() + 1, min=1)
    ijk = torch.minimum(((pts - lo) / cell).floor().long(), dims - 1).clamp_min(0)
    cid = (ijk[:, 0] * dims[1] + ijk[:, 1]) * dims[2] + ijk[:, 2]
    order = torch.argsort(cid)
    sorted_pts = pts[order].contiguous()
    ncell = int(dims.prod().item())
    counts = torch.bincount(cid, minlength=ncell)
    cell_start = torch.zeros(ncell + 1, dtype=torch.int32, device=dev)
    cell_start[1:] = torch.cumsum(counts, 0).to(torch.int32)
    g = RgsKnnGrid()
    g.lo[:] = lo.tolist()
    g.cell = cell
    g.dims[:] = [int(v) for v in dims.tolist()]
    res = torch.empty(P, dtype=torch.float32, device=dev)
    native.call("knn3", dev, g, sorted_pts, cell_start, P, res, sig="pppipp")
    out = torch.empty_like(res)
    out[order] = res
    return out
