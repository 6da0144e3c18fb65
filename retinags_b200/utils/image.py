"""Image files and image metrics.

PNG/JPEG decoding goes through Pillow when it is importable; PNG writing has a dependency-free zlib
fallback so that evaluation images can be dumped on a bare compute box.  ``psnr`` follows
``utils/image_utils.py:17-19`` of the reference.
"""
from __future__ import annotations

import struct
import zlib

import numpy as np
import torch


def psnr(img1: torch.Tensor, img2: torch.Tensor) -> torch.Tensor:
    mse = ((img1 - img2) ** 2).reshape(img1.shape[0], -1).mean(1, keepdim=True)
    return 20 * torch.log10(1.0 / torch.sqrt(mse))


def psnr_from_mse(mse: float) -> float:
    import math
    return 20.0 * math.log10(1.0 / math.sqrt(max(mse, 1e-20)))


def _to_uint8_hwc(img: torch.Tensor) -> np.ndarray:
    a = img.detach().float().cpu().clamp(0, 1)
    if a.dim() == 3 and a.shape[0] in (1, 3, 4):
        a = a.permute(1, 2, 0)
    return (a * 255.0 + 0.5).to(torch.uint8).numpy()


def save_png(path: str, img: torch.Tensor):
    """Write a (3,H,W) or (H,W,3) float image in [0,1] as an 8-bit PNG."""
    arr = _to_uint8_hwc(img)
    try:
        from PIL import Image
        Image.fromarray(arr.squeeze(-1) if arr.shape[-1] == 1 else arr).save(path)
        return
    except ImportError:
        pass
    h, w, c = arr.shape
    color_type = {1: 0, 3: 2, 4: 6}[c]
    raw = b"".join(b"\x00" + arr[y].tobytes() for y in range(h))

    def chunk(tag, data):
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)

    with open(path, "wb") as f:
        f.write(b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, color_type, 0, 0, 0))
                + chunk(b"IDAT", zlib.compress(raw, 3)) + chunk(b"IEND", b""))


def load_image(path: str, resolution: tuple[int, int] | None = None, white_background: bool = False) -> torch.Tensor:
    """(3,H,W) float32 in [0,1]; RGBA is composited over black or white; optional (W,H) resize."""
    from PIL import Image
    im = Image.open(path)
    if resolution is not None and tuple(im.size) != tuple(resolution):
        im = im.resize(resolution)
    a = torch.from_numpy(np.array(im)).float() / 255.0
    if a.dim() == 2:
        a = a[..., None].expand(-1, -1, 3)
    if a.shape[-1] == 4:
        bg = 1.0 if white_background else 0.0
        a = a[..., :3] * a[..., 3:4] + bg * (1 - a[..., 3:4])
    return a[..., :3].permute(2, 0, 1).contiguous()
