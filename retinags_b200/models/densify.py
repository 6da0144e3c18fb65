"""Adaptive density control on a :class:`GaussianStore`.

Same rules as the reference (``scene/gaussian_nn_module.py:689-751,1002-1036``): clone small
Gaussians and split large ones whose average screen-space gradient reaches the threshold (a split
draws N=2 samples from the Gaussian itself and shrinks the scale by 1/(0.8 N)); prune transparent,
screen-filling and world-oversized ones; new Gaussians start with zero Adam moments; all statistics
restart afterwards.  Differences: everything runs on the store's device (the reference samples the
split offsets on the CPU, ``:707-708``), and the parameter/moment surgery is one gather per buffer
instead of per-tensor optimizer rewrites (``:589-664``).
"""
from __future__ import annotations

import torch

from .gaussians import NAMES, GaussianStore


def _rotation_matrices(q: torch.Tensor) -> torch.Tensor:
    q = q / q.norm(dim=1, keepdim=True)
    r, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    R = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - r * z), 2 * (x * z + r * y),
                     2 * (x * y + r * z), 1 - 2 * (x * x + z * z), 2 * (y * z - r * x),
                     2 * (x * z - r * y), 2 * (y * z + r * x), 1 - 2 * (x * x + y * y)], dim=-1)
    return R.view(-1, 3, 3)


def densify_and_prune(store: GaussianStore, max_grad: float, min_opacity: float, extent: float,
                      max_screen_size: float | None, percent_dense: float = 0.01, max_size: int | None = None,
                      skip_prune: bool = False, skip_clone: bool = False, skip_split: bool = False,
                      generator: torch.Generator | None = None, n_split: int = 2) -> dict:
    n0 = store.count
    info = dict(cloned=0, split=0, pruned=0)
    if n0 == 0:
        return info
    over = max_size is not None and n0 > max_size
    if not over:
        grads = store.grad_accum[:n0] / store.denom[:n0]
        grads = torch.nan_to_num(grads, nan=0.0, posinf=0.0, neginf=0.0)
        p = store.views()
        max_scale = torch.exp(p["scale"]).max(dim=1).values
        hot = grads >= max_grad
        sel_clone = hot & (max_scale <= percent_dense * extent)
        sel_split = hot & (max_scale > percent_dense * extent)
        new = []
        if not skip_clone and bool(sel_clone.any()):
            idx = sel_clone.nonzero(as_tuple=True)[0]
            new.append({k: p[k][idx].clone() for k in NAMES})
            info["cloned"] = int(idx.numel())
        split_idx = None
        if not skip_split and bool(sel_split.any()):
            split_idx = sel_split.nonzero(as_tuple=True)[0]
            k = int(split_idx.numel())
            stds = torch.exp(p["scale"][split_idx]).repeat(n_split, 1)
            samples = torch.randn(stds.shape, device=store.device, generator=generator) * stds
            rots = _rotation_matrices(p["rot"][split_idx]).repeat(n_split, 1, 1)
            xyz = torch.bmm(rots, samples.unsqueeze(-1)).squeeze(-1) + p["xyz"][split_idx].repeat(n_split, 1)
            new.append(dict(xyz=xyz, sh=p["sh"][split_idx].repeat(n_split, 1),
                            scale=torch.log(stds / (0.8 * n_split)), rot=p["rot"][split_idx].repeat(n_split, 1),
                            opacity=p["opacity"][split_idx].repeat(n_split, 1)))
            info["split"] = k
        for g in new:
            store.append_new(g)
        if split_idx is not None:
            keep = torch.ones(store.count, dtype=torch.bool, device=store.device)
            keep[split_idx] = False
            store.keep(keep)
    if not skip_prune and store.count:
        p = store.views()
        prune = torch.sigmoid(p["opacity"]).squeeze(1) < min_opacity
        if max_screen_size:
            prune |= store.max_radii[:store.count] > max_screen_size
            prune |= torch.exp(p["scale"]).max(dim=1).values > 0.1 * extent
        info["pruned"] = int(prune.sum())
        if info["pruned"]:
            store.keep(~prune)
    store.reset_stats()
    return info


def reset_opacity(store: GaussianStore, ceiling: float = 0.01):
    """Clamp opacities to ``ceiling`` and forget their Adam moments (``gaussian_nn_module.py:515-519``)."""
    if store.count == 0:
        return
    p = store.views()
    o = torch.minimum(torch.sigmoid(p["opacity"]), torch.full_like(p["opacity"], ceiling))
    p["opacity"].copy_(torch.log(o / (1 - o)))
    store.views("exp_avg")["opacity"].zero_()
    store.views("exp_avg_sq")["opacity"].zero_()


def discard_out_of_range(store: GaussianStore, scale_factor: float = 1.0):
    """Drop Gaussians whose 3-sigma extent misses the store's box (``gaussian_nn_module.py:1028-1036``)."""
    if store.count == 0:
        return
    p = store.views()
    r = (3.0 * scale_factor * torch.exp(p["scale"]).max(dim=1, keepdim=True).values).clamp_min(0)
    lo = torch.as_tensor(store.box_lo, dtype=torch.float32, device=store.device)
    hi = torch.as_tensor(store.box_hi, dtype=torch.float32, device=store.device)
    keep = ((p["xyz"] + r >= lo) & (p["xyz"] - r <= hi)).all(dim=1)
    store.keep(keep)
