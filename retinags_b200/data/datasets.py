"""Camera datasets.

Parity: ``utils/datasets.py:25-187`` (``CameraListDataset``, ``DatasetRepeater``, ``GroupedItems``) and
the resolution rule of ``utils/camera_utils.py:20-78`` (``-r`` in {1,2,4,8} divides, ``-1`` caps the
width at 1600, any other value is the target width).  The reference decodes the image file on every
access; here decoded images are cached in pinned host memory (bounded by ``cache_bytes``), so later
epochs only pay the host->device copy of the rows a rank owns.
"""
from __future__ import annotations

import threading

import torch
from torch.utils.data import Dataset

from .cameras import Camera


def target_resolution(orig_w: int, orig_h: int, resolution, resolution_scale: float = 1.0) -> tuple[int, int]:
    if resolution in (1, 2, 4, 8):
        return round(orig_w / (resolution_scale * resolution)), round(orig_h / (resolution_scale * resolution))
    if resolution == -1:
        down = orig_w / 1600 if orig_w > 1600 else 1.0
    else:
        down = orig_w / resolution
    scale = float(down) * float(resolution_scale)
    return int(orig_w / scale), int(orig_h / scale)


class CameraListDataset(Dataset):
    def __init__(self, cam_infos: list, resolution=-1, resolution_scale: float = 1.0, white_background: bool = False,
                 pin: bool = True, cache_bytes: int = 64 << 30):
        self.infos = list(cam_infos)
        self.resolution, self.resolution_scale = resolution, resolution_scale
        self.white_background = white_background
        self.pin = pin and torch.cuda.is_available()
        self.cache_bytes = cache_bytes
        self._cache: dict[int, torch.Tensor] = {}
        self._cached = 0
        self._lock = threading.Lock()  # items may be fetched by the prefetch threads (data/prefetch.py)

    def __len__(self):
        return len(self.infos)

    def _size(self, info) -> tuple[int, int]:
        return target_resolution(info.width, info.height, self.resolution, self.resolution_scale)

    def empty_item(self, idx: int) -> Camera:
        """Camera without pixels (what ranks that own no rows of the image need)."""
        info = self.infos[idx]
        if isinstance(info, Camera):
            return info.without_image()
        w, h = self._size(info)
        return Camera(uid=idx, R=info.R, T=info.T, fovx=info.fovx, fovy=info.fovy, width=w, height=h,
                      image_name=info.image_name, colmap_id=info.uid)

    def __getitem__(self, idx: int) -> Camera:
        info = self.infos[idx]
        if isinstance(info, Camera):  # synthetic scenes carry their pixels already
            return info
        cam = self.empty_item(idx)
        img = self._cache.get(idx)
        if img is None:
            from ..utils.image import load_image
            img = load_image(info.image_path, (cam.width, cam.height), self.white_background)
            if self.pin:
                img = img.pin_memory()
            nbytes = img.numel() * 4
            with self._lock:
                if idx not in self._cache and self._cached + nbytes <= self.cache_bytes:
                    self._cache[idx] = img
                    self._cached += nbytes
        cam.image = img
        return cam


class DatasetRepeater(Dataset):
    """``len`` samples drawn with a fixed stride from ``origin`` (``utils/datasets.py:122-141``)."""

    def __init__(self, origin: Dataset, repeat_utill: int, empty: bool = False, step: int = 1):
        self.origin, self.n, self.empty, self.step = origin, repeat_utill, empty, step

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        j = (idx * self.step) % len(self.origin)
        return self.origin.empty_item(j) if self.empty else self.origin[j]


class GroupedItems(Dataset):
    """Dataset of batches: item ``i`` is (indices, cameras) of group ``i`` (``utils/datasets.py:170-186``)."""

    def __init__(self, origin: CameraListDataset, groups: list[tuple], owner_fn=None):
        self.origin, self.groups, self.owner_fn = origin, list(groups), owner_fn

    def __len__(self):
        return len(self.groups)

    def __getitem__(self, i):
        ids = self.groups[i]
        return ids, [self.origin[j] for j in ids]
