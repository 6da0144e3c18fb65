"""Seeded synthetic scenes (Gaussians + cameras) for tests and benchmarks.

There is no counterpart in the reference, which only reads captured datasets
(``scene/dataset_readers.py``).  The generators produce the shapes used for benchmarking:

* ``uniform_scene``     Gaussians uniform in a cube, ring cameras (small plumbing scenes)
* ``cluster_scene``     mixture of anisotropic 3D clusters in a box, hemisphere cameras
* ``aerial_scene``      ground plane + vertical building-like clusters, downward-looking grid cameras

All parameters are *raw* (log-scale, logit-opacity, unnormalised quaternion), in the layout of the
parameter store: xyz (P,3), sh (P,48) coefficient-major, scale (P,3), rot (P,4), opacity (P,1).
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..utils import graphics
from .cameras import Camera


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def random_gaussians(n: int, means: torch.Tensor, seed: int, device="cpu", sh_degree: int = 3,
                     log_scale_mean: float = -4.0, log_scale_std: float = 0.5, dc_mean: float = 0.5,
                     dc_std: float = 0.2, rest_std: float = 0.2, opacity_mean: float = 0.0) -> dict:
    g = _gen(seed, device)
    kw = dict(device=device, dtype=torch.float32, generator=g)
    sh = torch.zeros(n, 16, 3, device=device)
    sh[:, 0] = dc_mean + dc_std * torch.randn(n, 3, **kw)
    nc = (sh_degree + 1) ** 2
    if nc > 1:
        sh[:, 1:nc] = rest_std * torch.randn(n, nc - 1, 3, **kw)
    scale = log_scale_mean + log_scale_std * torch.randn(n, 3, **kw)
    rot = torch.randn(n, 4, **kw)
    rot = rot / rot.norm(dim=1, keepdim=True)
    opacity = opacity_mean + torch.randn(n, 1, **kw)
    return dict(xyz=means.contiguous(), sh=sh.view(n, 48).contiguous(), scale=scale, rot=rot, opacity=opacity)


def uniform_gaussians(n: int, seed: int, device="cpu", sh_degree: int = 1, half: float = 1.0, **kw) -> dict:
    g = _gen(seed + 17, device)
    means = (torch.rand(n, 3, device=device, generator=g) * 2 - 1) * half
    return random_gaussians(n, means, seed, device, sh_degree, **kw)


def cluster_means(n: int, seed: int, device="cpu", n_clusters: int = 64, box: float = 20.0) -> torch.Tensor:
    """Mixture of ``n_clusters`` anisotropic 3D Gaussians inside a ``box``-unit cube centred at 0."""
    g = _gen(seed + 101, device)
    centers = (torch.rand(n_clusters, 3, device=device, generator=g) - 0.5) * box * 0.8
    centers[:, 2] = centers[:, 2].abs() * 0.5  # clusters sit above the ground plane
    axes = 0.3 + 1.7 * torch.rand(n_clusters, 3, device=device, generator=g)
    rot = torch.randn(n_clusters, 3, 3, device=device, generator=g)
    q, _ = torch.linalg.qr(rot)
    which = torch.randint(0, n_clusters, (n,), device=device, generator=g)
    local = torch.randn(n, 3, device=device, generator=g) * axes[which]
    pts = torch.einsum("nij,nj->ni", q[which], local) + centers[which]
    return pts.clamp_(-box / 2, box / 2)


def cluster_gaussians(n: int, seed: int, device="cpu", sh_degree: int = 3, box: float = 20.0, **kw) -> dict:
    return random_gaussians(n, cluster_means(n, seed, device, box=box), seed, device, sh_degree, **kw)


def aerial_gaussians(n: int, seed: int, device="cpu", sh_degree: int = 3, extent: float = 2000.0,
                     n_buildings: int = 4096) -> dict:
    g = _gen(seed + 211, device)
    n_ground = n // 2
    ground = torch.empty(n_ground, 3, device=device)
    ground[:, :2] = (torch.rand(n_ground, 2, device=device, generator=g) - 0.5) * extent
    ground[:, 2] = -15.0 * torch.log(torch.rand(n_ground, device=device, generator=g).clamp_min(1e-6)) * 0.2
    nb = n - n_ground
    bc = (torch.rand(n_buildings, 2, device=device, generator=g) - 0.5) * extent
    bh = 10.0 + 60.0 * torch.rand(n_buildings, device=device, generator=g)
    bw = 5.0 + 20.0 * torch.rand(n_buildings, 2, device=device, generator=g)
    which = torch.randint(0, n_buildings, (nb,), device=device, generator=g)
    b = torch.empty(nb, 3, device=device)
    b[:, :2] = bc[which] + (torch.rand(nb, 2, device=device, generator=g) - 0.5) * bw[which]
    b[:, 2] = torch.rand(nb, device=device, generator=g) * bh[which]
    means = torch.cat([ground, b], dim=0)
    return random_gaussians(n, means, seed, device, sh_degree, log_scale_mean=-1.0)


def ring_cameras(n: int, radius: float, width: int, height: int, fov_deg: float = 60.0, z: float = 0.0) -> list[Camera]:
    cams = []
    fovx = math.radians(fov_deg)
    fovy = graphics.focal2fov(graphics.fov2focal(fovx, width), height)
    for i in range(n):
        a = 2 * math.pi * i / n
        eye = np.array([radius * math.cos(a), radius * math.sin(a), z])
        R, t = graphics.look_at(eye, np.zeros(3))
        cams.append(Camera(uid=i, R=R, T=t, fovx=fovx, fovy=fovy, width=width, height=height, image_name=f"ring_{i:04d}"))
    return cams


def hemisphere_cameras(n: int, radius: float, width: int, height: int, fov_deg: float = 50.0, seed: int = 0,
                       target=(0.0, 0.0, 1.0)) -> list[Camera]:
    """``n`` cameras on a Fibonacci-spiral hemisphere of the given radius, looking at ``target``."""
    cams = []
    fovx = math.radians(fov_deg)
    fovy = graphics.focal2fov(graphics.fov2focal(fovx, width), height)
    golden = math.pi * (3.0 - math.sqrt(5.0))
    for i in range(n):
        zf = 0.15 + 0.8 * (i + 0.5) / n  # elevation from 0.15 to 0.95 of the radius
        r = math.sqrt(max(0.0, 1.0 - zf * zf))
        a = golden * i + 0.37 * seed
        eye = np.array([radius * r * math.cos(a), radius * r * math.sin(a), radius * zf])
        R, t = graphics.look_at(eye, np.asarray(target, dtype=np.float64))
        cams.append(Camera(uid=i, R=R, T=t, fovx=fovx, fovy=fovy, width=width, height=height, image_name=f"hemi_{i:04d}"))
    return cams


def aerial_cameras(n: int, extent: float, width: int, height: int, fov_deg: float = 60.0, seed: int = 0) -> list[Camera]:
    rng = np.random.default_rng(seed + 5)
    side = int(math.ceil(math.sqrt(n)))
    fovx = math.radians(fov_deg)
    fovy = graphics.focal2fov(graphics.fov2focal(fovx, width), height)
    cams = []
    for i in range(n):
        gx, gy = i % side, i // side
        eye = np.array([(gx + 0.5) / side - 0.5, (gy + 0.5) / side - 0.5, 0.0]) * extent * 0.9
        eye[2] = rng.uniform(150.0, 400.0)
        tilt = math.radians(rng.uniform(45.0, 90.0))
        heading = rng.uniform(0, 2 * math.pi)
        d = np.array([math.cos(heading) * math.cos(tilt), math.sin(heading) * math.cos(tilt), -math.sin(tilt)])
        R, t = graphics.look_at(eye, eye + d, up=(0.0, 0.0, 1.0) if tilt < 1.55 else (0.0, 1.0, 0.0))
        cams.append(Camera(uid=i, R=R, T=t, fovx=fovx, fovy=fovy, width=width, height=height, zfar=2000.0,
                           image_name=f"aerial_{i:04d}"))
    return cams
