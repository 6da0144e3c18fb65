"""Shared scene builders for the tests."""
import torch

from retinags_b200.data import synthetic
from retinags_b200.ops import oracle, rasterize


def small_scene(n=600, seed=3, width=64, height=48, sh_degree=3, device="cpu", log_scale_mean=-2.6):
    g = synthetic.uniform_gaussians(n, seed, device=device, sh_degree=sh_degree, log_scale_mean=log_scale_mean)
    cams = synthetic.ring_cameras(4, 3.0, width, height)
    return g, cams


def activated(g):
    return dict(xyz=g["xyz"], sh=g["sh"], scale=torch.exp(g["scale"]),
                rot=g["rot"] / g["rot"].norm(dim=1, keepdim=True), opacity=torch.sigmoid(g["opacity"]))


def native_render(g, cam, sh_degree, box=(None, None), raw=True, tight=True, device="cpu", want_depth=False,
                  binning="depth_first"):
    seg = rasterize.Segment(*(g[k].to(device).contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
    task = rasterize.RenderTask(device, binning=binning)
    c = rasterize.make_camera(cam, sh_degree, box[0], box[1], raw_params=raw, tight_rect=tight)
    out = task.forward(c, [seg], want_depth=want_depth, check=True)
    return out, task, seg, c


def oracle_render(g, cam, sh_degree, box=(None, None)):
    a = activated(g)
    return oracle.rasterize(cam, a["xyz"], a["sh"].view(-1, 16, 3), a["opacity"], a["scale"], a["rot"], sh_degree,
                            box[0], box[1])


def assert_mostly_close(a, b, atol, rtol, max_frac=2e-4, hard_atol=5e-3):
    """Element-wise closeness that tolerates a handful of pixels where the T < 1e-4 stop rule or the 1/255
    alpha reject flips between two float evaluation orders (FMA contraction differs between nvcc and g++)."""
    diff = (a - b).abs()
    bad = diff > (atol + rtol * b.abs())
    assert bad.float().mean().item() <= max_frac, f"{int(bad.sum())} of {bad.numel()} elements differ"
    assert diff.max().item() <= hard_atol, f"max abs diff {diff.max().item()}"
