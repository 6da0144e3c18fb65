"""Adaptive density control on a :class:`GaussianStore`.

Same rules as the reference (``scene/gaussian_nn_module.py:689-751,1002-1036``): clone small
Gaussians and split large ones whose average screen-space gradient reaches the threshold (a split
draws N=2 samples from the Gaussian itself and shrinks the scale by 1/(0.8 N)); prune transparent,
screen-filling and world-oversized ones; new Gaussians start with zero Adam moments; all statistics
restart afterwards.  Differences: everything runs on the store's device (the reference samples the
split offsets on the CPU, ``:707-708``), and the parameter/moment surgery is one gather per buffer
instead of per-tensor optimizer rewrites (``:589-664``).

Two implementations with the same decisions and the same output order (kept originals, clones, first
split children, second split children):

* :func:`densify_and_prune` with ``native=True`` (default): the classification, scan and compaction
  kernels of ``csrc/rgs_surgery.cu`` (CPU twin in ``csrc/rgs_cpu.cpp``), split offsets from a
  counter-based Philox generator keyed by ``(seed, row, child)``; parameters and moments are written once
  into fresh buffers;
* ``native=False``: the same rules in PyTorch operations (``torch.randn`` split offsets); it is the
  oracle of the kernels and the fallback when the device cannot hold a second copy of the state.
"""
from __future__ import annotations

import torch

from ..ops import native
from .gaussians import NAMES, RECORD, GaussianStore, _round_cap


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
                      generator: torch.Generator | None = None, n_split: int = 2, native_path: bool | None = None,
                      seed: int | None = None) -> dict:
    n0 = store.count
    info = dict(cloned=0, split=0, pruned=0)
    if n0 == 0:
        return info
    if native_path is None:
        native_path = n_split == 2 and _fits_twice(store)
    if native_path:
        return _densify_native(store, max_grad, min_opacity, extent, max_screen_size, percent_dense, max_size, skip_prune,
                               skip_clone, skip_split, generator, seed)
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


def _fits_twice(store: GaussianStore) -> bool:
    """The compaction kernels write a second copy of parameters and moments before the old one is released."""
    if store.device.type != "cuda":
        return True
    free, _ = torch.cuda.mem_get_info(store.device)
    # the gradient buffer is released first, so that only two more buffers are needed
    return free > 2.6 * RECORD * 4 * store.cap * 1.3


def _densify_native(store: GaussianStore, max_grad, min_opacity, extent, max_screen_size, percent_dense, max_size, skip_prune,
                    skip_clone, skip_split, generator, seed) -> dict:
    n0, dev = store.count, store.device
    if seed is None:
        seed = int(torch.randint(0, 2 ** 62, (1,), generator=generator if generator is not None and
                                 generator.device.type == "cpu" else None).item())
    cfg = native.RgsDensifyCfg(float(max_grad), float(percent_dense * extent), float(min_opacity),
                               float(max_screen_size) if max_screen_size else 0.0, float(0.1 * extent), int(skip_clone),
                               int(skip_split), int(skip_prune), int(max_size is not None and n0 > max_size), seed)
    nblocks = -(-n0 // native.SURGERY_BLOCK)
    codes = torch.empty(n0, dtype=torch.uint8, device=dev)
    offsets = torch.empty(4 * nblocks, dtype=torch.int32, device=dev)
    totals = torch.zeros(4, dtype=torch.int64, device=dev)
    native.call("densify_classify", dev, store.params, store.cap, n0, store.grad_accum, store.denom, store.max_radii, cfg,
                codes, offsets, totals)
    kept, cloned, child_a, child_b = (int(x) for x in totals.cpu())
    n1 = kept + cloned + child_a + child_b
    new_cap = _round_cap(max(n1, 4))
    if new_cap < store.cap and n1 > 0.5 * store.cap:
        new_cap = store.cap  # keep the capacity when the model did not shrink much: later growth needs no reallocation
    store.grads = None  # gradients do not survive surgery; released first to bound the peak
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    new = [torch.zeros(RECORD * new_cap, dtype=torch.float32, device=dev) for _ in range(3)]
    native.call("densify_gather", dev, store.params, store.exp_avg, store.exp_avg_sq, store.cap, n0, codes, offsets, totals,
                new[0], new[1], new[2], new_cap, seed, status)
    if int(status.item()) != 0:
        raise RuntimeError("densify_gather: destination smaller than the new model")
    store.adopt(new[0], new[1], new[2], new_cap, n1, with_moments=kept)
    # both children of a split exist or neither; "pruned" counts the originals that disappeared without a split
    return dict(cloned=cloned, split=child_a, pruned=n0 - kept - child_a)


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
