"""LPIPS (learned perceptual image patch similarity) with VGG-16 features, from local weight files.

The reference evaluates LPIPS through its vendored ``lpipsPyTorch`` package, which downloads the torchvision VGG-16
weights and the linear heads from the network every time it is constructed (``lpipsPyTorch/modules/utils.py:11-20``,
``networks.py:92``) and builds a new module per image (``lpipsPyTorch/__init__.py:19-21``).  Here the network is
written out in plain PyTorch and built once; the weights come from files the user provides:

* ``<dir>/vgg16.pth``    torchvision's VGG-16 state dict (keys ``features.<n>.weight|bias``) or only its ``features``
* ``<dir>/lpips_vgg.pth`` the five 1x1 heads of LPIPS v0.1 (keys ``lin<k>.model.1.weight``)

Without them :func:`load_lpips` returns ``None`` and the evaluation reports LPIPS as NaN.
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn
import torch.nn.functional as F

_VGG_CFG = (64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512)
_TAPS = (3, 8, 15, 22, 29)          # indices of relu1_2, relu2_2, relu3_3, relu4_3, relu5_3 in torchvision's features
_CHANNELS = (64, 128, 256, 512, 512)


def _vgg16_features() -> nn.Sequential:
    layers, c = [], 3
    for v in _VGG_CFG:
        if v == "M":
            layers.append(nn.MaxPool2d(2, 2))
        else:
            layers += [nn.Conv2d(c, v, 3, padding=1), nn.ReLU(inplace=False)]
            c = v
    return nn.Sequential(*layers)


class LPIPS(nn.Module):
    def __init__(self):
        super().__init__()
        self.features = _vgg16_features()
        self.lins = nn.ModuleList([nn.Conv2d(c, 1, 1, bias=False) for c in _CHANNELS])
        self.register_buffer("shift", torch.tensor([-0.030, -0.088, -0.188]).view(1, 3, 1, 1))
        self.register_buffer("scale", torch.tensor([0.458, 0.448, 0.450]).view(1, 3, 1, 1))
        for p in self.parameters():
            p.requires_grad_(False)

    def _taps(self, x: torch.Tensor) -> list[torch.Tensor]:
        out = []
        for i, layer in enumerate(self.features):
            x = layer(x)
            if i in _TAPS:
                out.append(x / (x.pow(2).sum(1, keepdim=True).sqrt() + 1e-10))
        return out

    @torch.no_grad()
    def forward(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """(N,) distances of image batches (N,3,H,W) (a single (3,H,W) image gives a scalar)."""
        single = a.dim() == 3
        if single:
            a, b = a[None], b[None]
        fa, fb = self._taps((a - self.shift) / self.scale), self._taps((b - self.shift) / self.scale)
        d = sum(lin((x - y) ** 2).mean(dim=(1, 2, 3)) for lin, x, y in zip(self.lins, fa, fb))
        return d[0] if single else d

    def load_weight_files(self, vgg_path: str, lin_path: str):
        sd = torch.load(vgg_path, map_location="cpu", weights_only=True)
        feats = {k[len("features."):]: v for k, v in sd.items() if k.startswith("features.")} or sd
        self.features.load_state_dict(feats)
        lin = torch.load(lin_path, map_location="cpu", weights_only=True)
        for k, conv in enumerate(self.lins):
            conv.weight.copy_(lin[f"lin{k}.model.1.weight"])
        return self


def load_lpips(weights_dir: str | None, device="cpu") -> LPIPS | None:
    """The metric with weights from ``weights_dir`` (or ``$RGS_LPIPS_WEIGHTS``), or None when the files are missing."""
    d = weights_dir or os.environ.get("RGS_LPIPS_WEIGHTS", "")
    vgg, lin = os.path.join(d, "vgg16.pth"), os.path.join(d, "lpips_vgg.pth")
    if not d or not (os.path.exists(vgg) and os.path.exists(lin)):
        return None
    return LPIPS().load_weight_files(vgg, lin).to(device).eval()
