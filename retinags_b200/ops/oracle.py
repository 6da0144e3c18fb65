"""Pure-PyTorch restatement of the half-Gaussian rasteriser, differentiable by autograd.

This is the correctness oracle of the native kernels (forward values and, through autograd, all
gradients) and needs nothing but ``torch``.  It restates, in tensor algebra, what the reference
computes in
``rasterization_kernels/diff-gaussian-rasterization-half-gaussian/cuda_rasterizer_hgs/forward.cu:20-405``
(SH colour, EWA projection with the 1.3*tan(fov) clamp and the 0.3 px low-pass, 3-sigma tile
rectangle, per-tile depth order, alpha clamp 0.99, 1/255 reject, ray-point-in-box clip, stop at
T < 1e-4).  Inputs are *activated* values, like the reference kernel's.
"""
from __future__ import annotations

import math

import torch

from ..data.cameras import Camera

SH_C0 = 0.28209479177387814
SH_C1 = 0.4886025119029199
SH_C2 = [1.0925484305920792, -1.0925484305920792, 0.31539156525252005, -1.0925484305920792, 0.5462742152960396]
SH_C3 = [-0.5900435899266435, 2.890611442640554, -0.4570457994644658, 0.3731763325901154, -0.4570457994644658,
         1.445305721320277, -0.5900435899266435]
TILE = 16


def eval_sh(deg: int, sh: torch.Tensor, dirs: torch.Tensor) -> torch.Tensor:
    """sh: (P,16,3) coefficient-major, dirs: (P,3) unit vectors -> (P,3) (before the +0.5 offset)."""
    x, y, z = dirs[:, 0:1], dirs[:, 1:2], dirs[:, 2:3]
    res = SH_C0 * sh[:, 0]
    if deg > 0:
        res = res - SH_C1 * y * sh[:, 1] + SH_C1 * z * sh[:, 2] - SH_C1 * x * sh[:, 3]
    if deg > 1:
        xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
        res = (res + SH_C2[0] * xy * sh[:, 4] + SH_C2[1] * yz * sh[:, 5] + SH_C2[2] * (2 * zz - xx - yy) * sh[:, 6]
               + SH_C2[3] * xz * sh[:, 7] + SH_C2[4] * (xx - yy) * sh[:, 8])
    if deg > 2:
        res = (res + SH_C3[0] * y * (3 * xx - yy) * sh[:, 9] + SH_C3[1] * xy * z * sh[:, 10]
               + SH_C3[2] * y * (4 * zz - xx - yy) * sh[:, 11] + SH_C3[3] * z * (2 * zz - 3 * xx - 3 * yy) * sh[:, 12]
               + SH_C3[4] * x * (4 * zz - xx - yy) * sh[:, 13] + SH_C3[5] * z * (xx - yy) * sh[:, 14]
               + SH_C3[6] * x * (xx - 3 * yy) * sh[:, 15])
    return res


def quat_to_rot(q: torch.Tensor) -> torch.Tensor:
    r, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    R = torch.stack([
        1 - 2 * (y * y + z * z), 2 * (x * y - r * z), 2 * (x * z + r * y),
        2 * (x * y + r * z), 1 - 2 * (x * x + z * z), 2 * (y * z - r * x),
        2 * (x * z - r * y), 2 * (y * z + r * x), 1 - 2 * (x * x + y * y)], dim=-1)
    return R.view(-1, 3, 3)


def project(cam: Camera, means3D, shs, opacities, scales, rotations, sh_degree: int, scale_modifier: float = 1.0):
    """Per-Gaussian projection. Returns dict of tensors over all P Gaussians plus a validity mask."""
    dt = means3D.dtype
    view = torch.as_tensor(cam.world_view_transform, dtype=dt)  # transposed storage: row-vector convention
    full = torch.as_tensor(cam.full_proj_transform, dtype=dt)
    W, H = cam.width, cam.height
    tfx, tfy = cam.tan_fovx, cam.tan_fovy
    fx, fy = W / (2 * tfx), H / (2 * tfy)
    ones = torch.ones_like(means3D[:, :1])
    ph = torch.cat([means3D, ones], dim=1)
    t = ph @ view  # (P,4) view space
    hom = ph @ full
    pw = 1.0 / (hom[:, 3] + 1e-7)
    ndc = hom[:, :2] * pw[:, None]
    px = ((ndc[:, 0] + 1.0) * W - 1.0) * 0.5
    py = ((ndc[:, 1] + 1.0) * H - 1.0) * 0.5
    tz = t[:, 2]
    valid = tz > 0.2
    tz_s = torch.where(valid, tz, torch.ones_like(tz))
    limx, limy = 1.3 * tfx, 1.3 * tfy
    txtz, tytz = t[:, 0] / tz_s, t[:, 1] / tz_s
    inx = (txtz >= -limx) & (txtz <= limx)
    iny = (tytz >= -limy) & (tytz <= limy)
    # the reference treats the clamped value as a constant in its backward
    txc = torch.where(inx, t[:, 0], (txtz.clamp(-limx, limx) * tz_s).detach())
    tyc = torch.where(iny, t[:, 1], (tytz.clamp(-limy, limy) * tz_s).detach())
    zero = torch.zeros_like(tz_s)
    J = torch.stack([fx / tz_s, zero, -(fx * txc) / (tz_s * tz_s), zero, fy / tz_s, -(fy * tyc) / (tz_s * tz_s)],
                    dim=-1).view(-1, 2, 3)
    Wrot = view[:3, :3].T  # world->view rotation
    M = J @ Wrot
    R = quat_to_rot(rotations)
    L = R * (scale_modifier * scales)[:, None, :]
    Sigma = L @ L.transpose(1, 2)
    cov = M @ Sigma @ M.transpose(1, 2)
    a = cov[:, 0, 0] + 0.3
    b = cov[:, 0, 1]
    c = cov[:, 1, 1] + 0.3
    det = a * c - b * b
    valid = valid & (det != 0)
    det_s = torch.where(det != 0, det, torch.ones_like(det))
    conic = torch.stack([c / det_s, -b / det_s, a / det_s], dim=-1)
    mid = 0.5 * (a + c)
    sq = torch.sqrt(torch.clamp(mid * mid - det, min=0.1))
    radius = torch.ceil(3.0 * torch.sqrt(torch.maximum(mid + sq, mid - sq))).detach()
    center = torch.as_tensor(cam.camera_center, dtype=dt)
    d = means3D - center
    d = d / d.norm(dim=1, keepdim=True)
    rgb_raw = eval_sh(sh_degree, shs, d) + 0.5
    rgb = torch.clamp_min(rgb_raw, 0.0)
    return dict(px=px, py=py, conic=conic, rgb=rgb, opacity=opacities.reshape(-1), w=hom[:, 3], depth=tz,
                radius=radius, valid=valid, cov_a=a, cov_c=c)


def rasterize(cam: Camera, means3D, shs, opacities, scales, rotations, sh_degree: int = 3,
              box_lo=None, box_hi=None, scale_modifier: float = 1.0):
    """Render one sub-model. Returns (C (3,H,W) premultiplied colour, T (H,W), D (H,W), info dict)."""
    dt = means3D.dtype
    W, H = cam.width, cam.height
    pr = project(cam, means3D, shs, opacities, scales, rotations, sh_degree, scale_modifier)
    tiles_x, tiles_y = (W + TILE - 1) // TILE, (H + TILE - 1) // TILE
    rad = pr["radius"]
    pxd, pyd = pr["px"].detach(), pr["py"].detach()

    def _clampi(v, hi):
        return torch.clamp(torch.trunc(v), 0, hi).to(torch.long)

    x0 = _clampi((pxd - rad) / TILE, tiles_x)
    y0 = _clampi((pyd - rad) / TILE, tiles_y)
    x1 = _clampi((pxd + rad + TILE - 1) / TILE, tiles_x)
    y1 = _clampi((pyd + rad + TILE - 1) / TILE, tiles_y)
    valid = pr["valid"] & ((x1 - x0) * (y1 - y0) > 0)
    c2w_t = torch.as_tensor(cam.view_world_transform, dtype=dt)
    lo = torch.as_tensor(box_lo if box_lo is not None else [-math.inf] * 3, dtype=dt)
    hi = torch.as_tensor(box_hi if box_hi is not None else [math.inf] * 3, dtype=dt)
    C = torch.zeros(3, H, W, dtype=dt)
    T = torch.ones(H, W, dtype=dt)
    D = torch.zeros(H, W, dtype=dt)
    depth_order = torch.argsort(pr["depth"].detach(), stable=True)
    radii = torch.where(valid, rad, torch.zeros_like(rad)).to(torch.int32)
    for ty in range(tiles_y):
        for tx in range(tiles_x):
            sel = valid & (x0 <= tx) & (x1 > tx) & (y0 <= ty) & (y1 > ty)
            ids = depth_order[sel[depth_order]]
            if ids.numel() == 0:
                continue
            ys = torch.arange(ty * TILE, min((ty + 1) * TILE, H))
            xs = torch.arange(tx * TILE, min((tx + 1) * TILE, W))
            gy, gx = torch.meshgrid(ys, xs, indexing="ij")
            pixx = gx.reshape(-1).to(dt)
            pixy = gy.reshape(-1).to(dt)
            dx = pr["px"][ids, None] - pixx[None]
            dy = pr["py"][ids, None] - pixy[None]
            con = pr["conic"][ids]
            power = -0.5 * (con[:, 0:1] * dx * dx + con[:, 2:3] * dy * dy) - con[:, 1:2] * dx * dy
            G = torch.exp(power)
            alpha = torch.clamp_max(pr["opacity"][ids, None] * G, 0.99)
            keep = (power <= 0) & (alpha >= 1.0 / 255.0)
            # half-Gaussian clip
            w = pr["w"][ids].detach()
            nx = ((2 * pixx + 1.0) / W - 1.0) * cam.tan_fovx
            ny = ((2 * pixy + 1.0) / H - 1.0) * cam.tan_fovy
            pv = torch.stack([nx[None] * (w[:, None] + 1e-7), ny[None] * (w[:, None] + 1e-7),
                              w[:, None].expand(-1, pixx.numel()), torch.ones(ids.numel(), pixx.numel(), dtype=dt)],
                             dim=-1)
            pwld = pv @ c2w_t
            inside = ((pwld[..., :3] > lo) & (pwld[..., :3] <= hi)).all(dim=-1)
            keep = keep & inside
            a_eff = torch.where(keep, alpha, torch.zeros_like(alpha))
            # stop rule: the first splat that would push T below 1e-4 ends the pixel
            T_incl = torch.cumprod(1 - a_eff, dim=0)
            stop = torch.cummax((T_incl < 1e-4).to(torch.int8), dim=0).values.bool()
            a_eff = torch.where(stop, torch.zeros_like(a_eff), a_eff)
            T_incl = torch.cumprod(1 - a_eff, dim=0)
            T_excl = torch.cat([torch.ones_like(T_incl[:1]), T_incl[:-1]], dim=0)
            wgt = a_eff * T_excl
            col = (wgt[:, :, None] * pr["rgb"][ids][:, None, :]).sum(0)  # (pix,3)
            dep = (wgt * pr["depth"][ids, None]).sum(0)
            hh, ww = ys.numel(), xs.numel()
            C[:, ys[0]:ys[0] + hh, xs[0]:xs[0] + ww] = col.T.reshape(3, hh, ww)
            T[ys[0]:ys[0] + hh, xs[0]:xs[0] + ww] = T_incl[-1].reshape(hh, ww)
            D[ys[0]:ys[0] + hh, xs[0]:xs[0] + ww] = dep.reshape(hh, ww)
    return C, T, D, dict(radii=radii, px=pr["px"], py=pr["py"])


def composite(partials_C, partials_T, bg):
    """Front-to-back over of partial images given in order. Returns (image (3,H,W), T_total)."""
    acc = torch.zeros_like(partials_C[0])
    t = torch.ones_like(partials_T[0])
    for Ck, Tk in zip(partials_C, partials_T):
        acc = acc + t[None] * Ck
        t = t * Tk
    bg = torch.as_tensor(bg, dtype=acc.dtype).view(3, 1, 1)
    return acc + bg * t[None], t


# the loss of the oracle is the PyTorch loss of utils/loss.py (one implementation: depthwise conv2d SSIM + L1)
from ..utils.loss import ssim, training_loss  # noqa: E402,F401


def gaussian_window(dtype=torch.float32):
    from ..utils.loss import gaussian_window as _gw
    return _gw(11, 1.5, dtype)
