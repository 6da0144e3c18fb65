"""Function-style render entry points.

Counterparts in the reference: ``gaussian_renderer/render.py:20-103`` (``render(viewpoint_camera, pc, pipe, bg_color,
scaling_modifier)`` of vanilla 3DGS, against the absent vanilla rasteriser), ``gaussian_renderer/render_half_gs.py:21-101``
(``render4BoundedGaussianModel``: one sub-model with its clip box).  Both return a dictionary with ``render``,
``viewspace_points``, ``visibility_filter``, ``radii`` (+ ``depth``/``alpha`` for the half-Gaussian variant).
Here they are thin wrappers over :class:`RenderTask`; they compute no gradients (training goes through
``GaussianModel.train_step`` / ``StepEngine.train_step``, autograd users through ``ops.rasterize.GaussianRasterizer``).
"""
from __future__ import annotations

import torch

from .models.gaussians import GaussianStore
from .ops.rasterize import RenderTask, make_camera


def render_submodel(camera, store: GaussianStore, bg_color=(0.0, 0.0, 0.0), scaling_modifier: float = 1.0,
                    want_depth: bool = True, clip_to_box: bool = True, task: RenderTask | None = None) -> dict:
    """Partial image of one sub-model: premultiplied colour + background * transmittance, depth, alpha = 1 - T."""
    task = task if task is not None else RenderTask(store.device)
    lo, hi = (store.box_lo, store.box_hi) if clip_to_box else (None, None)
    cam = make_camera(camera, store.active_sh_degree, lo, hi, raw_params=True)
    cam.scale_modifier = float(scaling_modifier)
    seg = store.segment(with_grads=False)
    out = task.forward(cam, [seg], want_depth=want_depth, check=True)  # (H,W,4): premultiplied RGB, T
    trans = out[..., 3]
    bg = torch.as_tensor(bg_color, dtype=torch.float32, device=out.device)
    image = (out[..., :3] + trans[..., None] * bg).permute(2, 0, 1).contiguous()
    radii = task.radii(0, [seg])
    return dict(render=image, alpha=(1.0 - trans)[None], depth=task.depth[None] if want_depth else None, radii=radii,
                visibility_filter=radii > 0, viewspace_points=None, partial=out)


def render(viewpoint_camera, pc, pipe=None, bg_color=(0.0, 0.0, 0.0), scaling_modifier: float = 1.0) -> dict:
    """Vanilla-3DGS signature; ``pc`` is a :class:`GaussianModel` (or a bare :class:`GaussianStore`)."""
    store = pc if isinstance(pc, GaussianStore) else pc.store
    return render_submodel(viewpoint_camera, store, bg_color, scaling_modifier, want_depth=False, clip_to_box=False)
