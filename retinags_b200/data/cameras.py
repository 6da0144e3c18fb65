"""Camera objects.

Parity: ``scene/cameras.py:21-111`` (``Camera``) and ``:350-433`` (``EmptyCamera``) of the
reference.  A camera carries world->view and full projection matrices in transposed storage, its
centre, and the view->world matrix (the reference calls it ``projection_matrix_inv`` although it
is C2W-transposed, ``scene/cameras.py:59-63``).  Ground-truth pixels live in pinned host memory
and are uploaded only by the rank that owns the image rows, instead of by every rank
(``parallel_utils/basic_parallel_trainer/trainer4tree_partition.py:330``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch

from ..utils import graphics


@dataclass
class Camera:
    uid: int
    R: np.ndarray  # camera-to-world rotation (3,3)
    T: np.ndarray  # world-to-view translation (3,)
    fovx: float
    fovy: float
    width: int
    height: int
    image_name: str = ""
    image: torch.Tensor | None = None  # (3,H,W) float32 on the host (pinned when possible)
    znear: float = 0.01
    zfar: float = 100.0
    trans: tuple = (0.0, 0.0, 0.0)
    scale: float = 1.0
    colmap_id: int = -1
    _cache: dict = field(default_factory=dict, repr=False)

    def _mats(self):
        if not self._cache:
            w2c = graphics.world_to_view(self.R, self.T, self.trans, self.scale)
            proj = graphics.projection_matrix(self.znear, self.zfar, self.fovx, self.fovy)
            self._cache["view_t"] = np.ascontiguousarray(w2c.T)
            self._cache["proj_t"] = np.ascontiguousarray(proj.T)
            self._cache["full_t"] = np.ascontiguousarray((w2c.T.astype(np.float64) @ proj.T.astype(np.float64))
                                                         .astype(np.float32))
            c2w = np.linalg.inv(w2c.astype(np.float64)).astype(np.float32)
            self._cache["c2w_t"] = np.ascontiguousarray(c2w.T)
            self._cache["center"] = c2w[:3, 3].copy()
        return self._cache

    @property
    def world_view_transform(self) -> np.ndarray:
        return self._mats()["view_t"]

    @property
    def projection_matrix(self) -> np.ndarray:
        return self._mats()["proj_t"]

    @property
    def full_proj_transform(self) -> np.ndarray:
        return self._mats()["full_t"]

    @property
    def view_world_transform(self) -> np.ndarray:
        return self._mats()["c2w_t"]

    @property
    def camera_center(self) -> np.ndarray:
        return self._mats()["center"]

    @property
    def tan_fovx(self) -> float:
        return math.tan(self.fovx * 0.5)

    @property
    def tan_fovy(self) -> float:
        return math.tan(self.fovy * 0.5)

    def pack(self) -> np.ndarray:
        """(16,4) package: rows 0-3 view, 4-7 full projection, 8-11 view->world, 12 = (W,H,fovx,fovy),
        13 = centre (layout of ``scene/cameras.py:80-93``)."""
        out = np.zeros((16, 4), dtype=np.float32)
        out[0:4] = self.world_view_transform
        out[4:8] = self.full_proj_transform
        out[8:12] = self.view_world_transform
        out[12] = (self.width, self.height, self.fovx, self.fovy)
        out[13, :3] = self.camera_center
        return out

    def without_image(self) -> "Camera":
        return Camera(self.uid, self.R, self.T, self.fovx, self.fovy, self.width, self.height, self.image_name,
                      None, self.znear, self.zfar, self.trans, self.scale, self.colmap_id)

    def to_json(self, idx: int) -> dict:
        """``cameras.json`` entry (``utils/camera_utils.py:101-121`` of the reference)."""
        Rt = np.eye(4)
        Rt[:3, :3] = self.R.T
        Rt[:3, 3] = self.T
        c2w = np.linalg.inv(Rt)
        return {
            "id": idx, "img_name": self.image_name, "width": self.width, "height": self.height,
            "position": c2w[:3, 3].tolist(), "rotation": [r.tolist() for r in c2w[:3, :3]],
            "fy": graphics.fov2focal(self.fovy, self.height), "fx": graphics.fov2focal(self.fovx, self.width),
        }
