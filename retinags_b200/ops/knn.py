"""Mean squared distance to the three nearest neighbours (initial Gaussian scale).

Stands in for ``simple_knn._C.distCUDA2`` which the reference imports from an absent submodule
(``scene/gaussian_nn_module.py:413-414``): ``scales = log(sqrt(clamp_min(dist2, 1e-7)))``.  Exact
search over a uniform grid of cells sized so that a cell holds a handful of points: candidates come
from the 27 neighbouring cells, and a point whose third neighbour lies farther than one cell is
re-examined against all points (rare, and only those points).  Runs on the device of ``points``.
"""
from __future__ import annotations

import torch


def _brute(q: torch.Tensor, pts: torch.Tensor, self_mask_offset: int | None, chunk: int = 4096) -> torch.Tensor:
    out = torch.empty(q.shape[0], device=q.device)
    for s in range(0, q.shape[0], chunk):
        d = torch.cdist(q[s:s + chunk].double(), pts.double()).pow(2).float()
        k = min(4, pts.shape[0])
        v = torch.topk(d, k, dim=1, largest=False).values
        v = v[:, 1:] if self_mask_offset is not None else v[:, :3]
        out[s:s + chunk] = v.mean(1) if v.shape[1] else 0.0
    return out


def knn3_dist2(points: torch.Tensor, per_cell: float = 6.0) -> torch.Tensor:
    """(P,3) -> (P,) mean of the squared distances to the 3 nearest other points."""
    P = points.shape[0]
    if P <= 4:
        return _brute(points, points, 0)
    if P <= 20000:
        return _brute(points, points, 0)
    dev = points.device
    lo, hi = points.min(0).values, points.max(0).values
    vol = torch.clamp(hi - lo, min=1e-6).prod().item()
    cell = (vol * per_cell / P) ** (1.0 / 3.0)
    dims = torch.clamp(((hi - lo) / cell).floor().long() + 1, min=1)
    ijk = torch.minimum(((points - lo) / cell).floor().long(), dims - 1)
    cid = (ijk[:, 0] * dims[1] + ijk[:, 1]) * dims[2] + ijk[:, 2]
    order = torch.argsort(cid)
    cid_s, pts_s = cid[order], points[order]
    ncell = int(dims.prod().item())
    counts = torch.bincount(cid_s, minlength=ncell)
    starts = torch.cumsum(counts, 0) - counts
    best = torch.full((P, 3), float("inf"), device=dev)
    idx_self = torch.arange(P, device=dev)
    ijk_s = ijk[order]
    max_cnt = int(counts.max().item())
    for dx in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dz in (-1, 0, 1):
                n = ijk_s + torch.tensor([dx, dy, dz], device=dev)
                ok = ((n >= 0) & (n < dims)).all(1)
                ncid = torch.where(ok, (n[:, 0] * dims[1] + n[:, 1]) * dims[2] + n[:, 2], torch.zeros_like(cid_s))
                s0 = starts[ncid]
                c0 = torch.where(ok, counts[ncid], torch.zeros_like(counts[ncid]))
                for j in range(max_cnt):
                    valid = j < c0
                    if not bool(valid.any()):
                        break
                    cand = torch.clamp(s0 + j, max=P - 1)
                    d = (pts_s - pts_s[cand]).pow(2).sum(1)
                    d = torch.where(valid & (cand != idx_self), d, torch.full_like(d, float("inf")))
                    best = torch.sort(torch.cat([best, d[:, None]], 1), dim=1).values[:, :3]
    # neighbours inside the 27 cells are exact when the third one is closer than the cell size
    redo = (best[:, 2] > cell * cell) | ~torch.isfinite(best[:, 2])
    res = best.mean(1)
    if bool(redo.any()):
        ridx = redo.nonzero(as_tuple=True)[0]
        d = _brute(pts_s[ridx], pts_s, 0)
        res[ridx] = d
    out = torch.empty(P, device=dev)
    out[order] = res
    return out
