"""Loss and metric functions in plain PyTorch.

Counterparts of the reference's ``utils/loss_utils.py:17-63`` (``l1_loss``, ``l2_loss``, ``ssim`` with the 11x11
sigma-1.5 window, zero padding, C1 = 0.01^2, C2 = 0.03^2) and ``utils/image_utils.py:14-19`` (``mse``, ``psnr``).
Training and evaluation use the fused kernels of ``csrc/rgs_loss.cu``; these are the readable definitions, the oracle
of the kernel tests, and what scripts call on arbitrary tensors (they are differentiable through autograd).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def l1_loss(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return (a - b).abs().mean()


def l2_loss(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return ((a - b) ** 2).mean()


def gaussian_window(size: int = 11, sigma: float = 1.5, dtype=torch.float32, device=None) -> torch.Tensor:
    g = torch.tensor([math.exp(-((i - size // 2) ** 2) / (2.0 * sigma * sigma)) for i in range(size)], dtype=dtype, device=device)
    return g / g.sum()


def ssim(img1: torch.Tensor, img2: torch.Tensor, window_size: int = 11, size_average: bool = True) -> torch.Tensor:
    """SSIM of (C,H,W) or (N,C,H,W) images, depthwise Gaussian window, zero padding."""
    squeeze = img1.dim() == 3
    if squeeze:
        img1, img2 = img1[None], img2[None]
    c = img1.shape[1]
    g = gaussian_window(window_size, 1.5, img1.dtype, img1.device)
    win = (g[:, None] * g[None, :]).expand(c, 1, window_size, window_size).contiguous()
    pad = window_size // 2
    mu1, mu2 = F.conv2d(img1, win, padding=pad, groups=c), F.conv2d(img2, win, padding=pad, groups=c)
    mu1_sq, mu2_sq, mu12 = mu1 * mu1, mu2 * mu2, mu1 * mu2
    s1 = F.conv2d(img1 * img1, win, padding=pad, groups=c) - mu1_sq
    s2 = F.conv2d(img2 * img2, win, padding=pad, groups=c) - mu2_sq
    s12 = F.conv2d(img1 * img2, win, padding=pad, groups=c) - mu12
    c1, c2 = 0.01 ** 2, 0.03 ** 2
    m = ((2 * mu12 + c1) * (2 * s12 + c2)) / ((mu1_sq + mu2_sq + c1) * (s1 + s2 + c2))
    return m.mean() if size_average else m.mean(dim=(1, 2, 3))


def mse(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return ((a - b) ** 2).reshape(a.shape[0], -1).mean(1, keepdim=True)


def psnr(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return 20.0 * torch.log10(1.0 / torch.sqrt(mse(a, b)))


def training_loss(image: torch.Tensor, gt: torch.Tensor, lambda_dssim: float = 0.2) -> torch.Tensor:
    """(1 - lambda) L1 + lambda (1 - SSIM), the loss of the trainer (``trainer4tree_partition.py:436-455``)."""
    return (1.0 - lambda_dssim) * l1_loss(image, gt) + lambda_dssim * (1.0 - ssim(image, gt))
