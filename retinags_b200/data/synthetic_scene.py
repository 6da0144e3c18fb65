"""Synthetic scenes for the trainer: ``--synthetic kind:key=value:...`` instead of ``-s``.

``kind`` is ``uniform`` (cube, ring cameras), ``cluster`` (cluster mixture, hemisphere cameras) or ``aerial``
(ground plane + buildings, downward grid cameras).  Keys: ``n`` target Gaussians that produce the ground-truth
images, ``w``/``h`` resolution, ``views`` training views, ``test`` test views, ``seed``, ``init`` number of
initial points handed to the trainer (sampled from the target's centres with their base colour).
"""
from __future__ import annotations

import torch

from ..ops.rasterize import RenderTask, Segment, make_camera
from . import synthetic
from .readers import SceneInfo, nerfpp_norm


def parse_spec(spec: str) -> tuple[str, dict]:
    parts = spec.split(":")
    kv = dict(n=20000, w=128, h=96, views=8, test=2, seed=0, init=0, deg=3)
    for p in parts[1:]:
        k, v = p.split("=")
        kv[k] = int(v)
    return parts[0], kv


def build_synthetic_scene(spec: str, mdp=None, device=None) -> SceneInfo:
    kind, kv = parse_spec(spec)
    device = device or (torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu"))
    n, seed = kv["n"], kv["seed"]
    total = kv["views"] + kv["test"]
    if kind == "uniform":
        g = synthetic.uniform_gaussians(n, seed + 1, device, sh_degree=kv["deg"])
        cams = synthetic.ring_cameras(total, 3.0, kv["w"], kv["h"], 60.0)
    elif kind == "cluster":
        g = synthetic.cluster_gaussians(n, seed + 1, device, sh_degree=kv["deg"])
        cams = synthetic.hemisphere_cameras(total, 8.0, kv["w"], kv["h"], 50.0, seed)
    elif kind == "aerial":
        g = synthetic.aerial_gaussians(n, seed + 1, device, sh_degree=kv["deg"])
        cams = synthetic.aerial_cameras(total, 2000.0, kv["w"], kv["h"], 60.0, seed)
    else:
        raise ValueError(f"unknown synthetic scene kind {kind!r}")
    seg = Segment(g["xyz"], g["sh"], g["scale"], g["rot"], g["opacity"])
    task = RenderTask(device)
    pin = torch.cuda.is_available()
    for cam in cams:
        out = task.forward(make_camera(cam, kv["deg"]), [seg], check=True)
        img = out[..., :3].permute(2, 0, 1).contiguous().cpu()
        cam.image = img.pin_memory() if pin else img
    n_init = kv["init"] or n
    sel = torch.randperm(n, generator=torch.Generator().manual_seed(seed))[:n_init]
    pts = g["xyz"].cpu()[sel].numpy()
    col = (g["sh"].cpu()[sel, :3] * 0.28209479177387814 + 0.5).clamp(0, 1).numpy()
    # test views are taken at a regular stride so that they cover the rig
    stride = max(total // max(kv["test"], 1), 1)
    test_idx = set(list(range(0, total, stride))[: kv["test"]])
    train = [c for i, c in enumerate(cams) if i not in test_idx]
    test = [c for i, c in enumerate(cams) if i in test_idx]
    for i, c in enumerate(train):
        c.uid = i
    for i, c in enumerate(test):
        c.uid = i
    return SceneInfo(pts, col, train, test, nerfpp_norm(train), "", f"synthetic:{kind}")
