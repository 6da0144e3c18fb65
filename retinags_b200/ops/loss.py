"""Compositing of partial images and the fused L1 + D-SSIM loss, through the native kernels.

``CompositeLoss`` owns the per-view buffers (composited image, total transmittance, SSIM derivative
maps, image gradient, loss sums) and exposes three steps, each restricted to a band of image rows
so that several ranks can each own a band of the same view:

1. ``composite``   ordered front-to-back "over" of K partial (H,W,4) images
2. ``loss``        L1 and SSIM statistics + derivative maps, then d(loss)/d(image)
3. ``backward``    d(loss)/d(partial_k) for every partial (dC_k = T_<k g, dT_k = T_<k S_k.g)

The reference performs 1 with ATen ops (``result_aggregator.py:244-259``), 2 with cuDNN
convolutions (``utils/loss_utils.py:17-63``) and leaves 3 and the backward of 2 to autograd.
The loss per image is ``(1-lambda) L1 + lambda (1 - SSIM)``; losses of the images of a batch are
summed (``trainer4tree_partition.py:450-454``).
"""
from __future__ import annotations

import ctypes

import torch

from . import native

import os

HALO = 5  # SSIM window radius
# statistics pass of SSIM on the tensor cores (csrc/rgs_ssim_tc.cu) instead of the fp32 SIMT kernel
USE_TENSOR_CORES = os.environ.get("RGS_SSIM_TC", "0") == "1"  # measured slower than the SIMT kernel: opt-in


class CompositeLoss:
    def __init__(self, device, H: int, W: int):
        self.device = torch.device(device)
        self.H, self.W = H, W
        dev = self.device
        self.image = torch.zeros(3, H, W, dtype=torch.float32, device=dev)
        self.trans = torch.ones(H, W, dtype=torch.float32, device=dev)
        self.dmaps = torch.zeros(9, H, W, dtype=torch.float32, device=dev)
        self.g_image = torch.zeros(3, H, W, dtype=torch.float32, device=dev)
        self.sums = torch.zeros(3, dtype=torch.float64, device=dev)
        self.status = torch.zeros(native.CNT_WORDS, dtype=torch.int32, device=dev)
        # the partials come from the blend kernels, whose transmittance carries a "pixel finished" mark in its lowest
        # mantissa bit: the backward then gives exactly zero to the partials behind a finished pixel (set by the engine;
        # off for partials of any other origin, whose low bits mean nothing)
        self.marked = False
        self.tensor_cores = USE_TENSOR_CORES and self.device.type == "cuda" and self._tc_supported()

    def _tc_supported(self) -> bool:
        import ctypes
        fn = native.lib("cuda").rgs_cuda_ssim_tc_supported
        fn.argtypes, fn.restype = [ctypes.c_int64, ctypes.c_int64], ctypes.c_int
        return bool(fn(self.H, self.W))

    def _ssim_fwd(self, gt, c0, c1, r0, r1):
        if self.tensor_cores:
            native.call("ssim_fwd_tc", self.device, self.image, gt, self.H, self.W, c0, c1, r0, r1, self.dmaps, self.sums,
                        self.status, sig="ppiiiiiipppp")
        else:
            native.call("ssim_fwd", self.device, self.image, gt, self.H, self.W, c0, c1, r0, r1, self.dmaps, self.sums)

    @staticmethod
    def _bg(bg):
        return (ctypes.c_float * 3)(*[float(v) for v in bg])

    def composite(self, partials: list[torch.Tensor], bg, row0: int = 0, row1: int | None = None, image=None, trans=None):
        """Composite rows [row0,row1) of the ordered partials into ``self.image`` / ``self.trans`` (or into the
        (3,H,W) / (H,W) buffers given)."""
        row1 = self.H if row1 is None else row1
        for p in partials:  # tensors, or raw (virtual full-height) base addresses
            assert isinstance(p, int) or (p.is_contiguous() and p.shape[-1] == 4)
        image = self.image if image is None else image
        trans = self.trans if trans is None else trans
        ptrs = native.pointer_array(partials)
        native.call("composite_fwd", self.device, ptrs, len(partials), self._bg(bg), self.H, self.W, row0, row1,
                    image, trans)
        return image, trans

    def loss(self, gt: torch.Tensor, lambda_dssim: float = 0.2, row0: int = 0, row1: int | None = None,
             weight: float = 1.0):
        """Loss statistics and d(loss)/d(image) for rows [row0,row1) of the composited image.

        The image must be composited on rows [row0-10, row1+10) (clipped to the image).  Returns the
        device tensor of accumulated sums (sum|d|, sum ssim, sum d^2) over the band; the loss value
        is ``loss_from_sums``.  ``weight`` scales the gradient (1 = summed per-image losses).
        """
        H, W = self.H, self.W
        row1 = H if row1 is None else row1
        assert gt.is_contiguous() and gt.shape == (3, H, W)
        c0, c1 = max(0, row0 - HALO), min(H, row1 + HALO)
        self.sums.zero_()
        self._ssim_fwd(gt, c0, c1, row0, row1)
        npx = 3.0 * H * W
        native.call("ssim_bwd", self.device, self.image, gt, self.dmaps, H, W, row0, row1, c0, c1,
                    weight * (1.0 - lambda_dssim) / npx, weight * lambda_dssim / npx, self.g_image)
        return self.sums

    def fused_loss_backward(self, partials, grads, gt: torch.Tensor, bg, lambda_dssim: float = 0.2, row0: int = 0,
                            row1: int | None = None, weight: float = 1.0):
        """Training path in two launches: composite + loss statistics, then d(loss)/d(partial_k) for every partial.

        Equivalent to ``composite`` on rows [row0-10, row1+10), ``loss`` and ``backward`` on rows [row0,row1); the
        partial slots must hold rows [row0-10, row1+10) (clipped to the image).  Returns the loss sums.
        """
        H, W = self.H, self.W
        row1 = H if row1 is None else row1
        assert gt.is_contiguous() and gt.shape == (3, H, W)
        if self.tensor_cores:  # the tensor-core statistics pass reads the composited image from memory
            self.composite(partials, bg, max(0, row0 - 2 * HALO), min(H, row1 + 2 * HALO))
            sums = self.loss(gt, lambda_dssim, row0, row1, weight)
            self.backward(partials, grads, bg, row0, row1)
            return sums
        c0, c1 = max(0, row0 - HALO), min(H, row1 + HALO)
        self.sums.zero_()
        pp, gp, bgc = native.pointer_array(partials), native.pointer_array(grads), self._bg(bg)
        native.call("composite_ssim_fwd", self.device, pp, len(partials), bgc, gt, H, W, c0, c1, row0, row1, self.image,
                    self.trans, self.dmaps, self.sums, sig="pippiiiiiippppp")
        npx = 3.0 * H * W
        native.call("ssim_composite_bwd", self.device, pp, gp, len(partials), bgc, self.image, gt, self.dmaps, H, W, row0, row1,
                    c0, c1, weight * (1.0 - lambda_dssim) / npx, weight * lambda_dssim / npx, self.g_image,
                    1 if self.marked else 0, sig="ppippppiiiiiiffpip")
        return self.sums

    def stats(self, gt: torch.Tensor, row0: int = 0, row1: int | None = None):
        """Loss statistics only (no gradient): accumulated (sum|d|, sum ssim, sum d^2) over rows [row0,row1)."""
        H, W = self.H, self.W
        row1 = H if row1 is None else row1
        c0, c1 = max(0, row0), min(H, row1)
        self.sums.zero_()
        self._ssim_fwd(gt, c0, c1, row0, row1)
        return self.sums

    def loss_from_sums(self, sums, lambda_dssim: float = 0.2) -> dict:
        s = sums.tolist() if isinstance(sums, torch.Tensor) else list(sums)
        npx = 3.0 * self.H * self.W
        l1, ssim, mse = s[0] / npx, s[1] / npx, s[2] / npx
        return dict(l1=l1, ssim=ssim, mse=mse, loss=(1.0 - lambda_dssim) * l1 + lambda_dssim * (1.0 - ssim))

    def backward(self, partials: list[torch.Tensor], grads: list[torch.Tensor], bg, row0: int = 0,
                 row1: int | None = None):
        """Write d(loss)/d(partial_k) on rows [row0,row1) into ``grads[k]`` ((H,W,4): dC, dT)."""
        row1 = self.H if row1 is None else row1
        pp = native.pointer_array(partials)
        gp = native.pointer_array(grads)
        native.call("composite_bwd", self.device, pp, gp, len(partials), self._bg(bg), self.H, self.W, row0, row1,
                    self.g_image, 1 if self.marked else 0)
