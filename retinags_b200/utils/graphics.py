"""Camera matrices in the storage convention of 3DGS (4x4 matrices kept transposed).

Behavioural parity: ``utils/graphics_utils.py:38-89`` of the reference (world-to-view with an
optional recentring, the z_sign=+1 perspective matrix with ``P[3,2] = 1``, fov/focal conversion).
"""
from __future__ import annotations

import math

import numpy as np


def world_to_view(R: np.ndarray, t: np.ndarray, translate=(0.0, 0.0, 0.0), scale: float = 1.0) -> np.ndarray:
    """4x4 world->view matrix. ``R`` is the camera-to-world rotation, ``t`` the world-to-view translation."""
    Rt = np.eye(4, dtype=np.float64)
    Rt[:3, :3] = np.asarray(R, dtype=np.float64).T
    Rt[:3, 3] = np.asarray(t, dtype=np.float64)
    c2w = np.linalg.inv(Rt)
    c2w[:3, 3] = (c2w[:3, 3] + np.asarray(translate, dtype=np.float64)) * scale
    return np.linalg.inv(c2w).astype(np.float32)


def view_to_world(R, t, translate=(0.0, 0.0, 0.0), scale: float = 1.0) -> np.ndarray:
    return np.linalg.inv(world_to_view(R, t, translate, scale).astype(np.float64)).astype(np.float32)


def projection_matrix(znear: float, zfar: float, fovx: float, fovy: float) -> np.ndarray:
    tx, ty = math.tan(fovx / 2), math.tan(fovy / 2)
    top, right = ty * znear, tx * znear
    P = np.zeros((4, 4), dtype=np.float32)
    P[0, 0] = 2.0 * znear / (2 * right)
    P[1, 1] = 2.0 * znear / (2 * top)
    P[3, 2] = 1.0
    P[2, 2] = zfar / (zfar - znear)
    P[2, 3] = -(zfar * znear) / (zfar - znear)
    return P


def fov2focal(fov: float, pixels: float) -> float:
    return pixels / (2 * math.tan(fov / 2))


def focal2fov(focal: float, pixels: float) -> float:
    return 2 * math.atan(pixels / (2 * focal))


def look_at(eye, target, up=(0.0, 0.0, 1.0)):
    """Camera-to-world rotation (columns = right, down, forward) and world-to-view translation."""
    eye = np.asarray(eye, dtype=np.float64)
    fwd = np.asarray(target, dtype=np.float64) - eye
    fwd /= np.linalg.norm(fwd)
    upv = np.asarray(up, dtype=np.float64)
    right = np.cross(fwd, upv)
    if np.linalg.norm(right) < 1e-8:
        right = np.cross(fwd, np.array([0.0, 1.0, 0.0]))
    right /= np.linalg.norm(right)
    down = np.cross(fwd, right)
    R = np.stack([right, down, fwd], axis=1)  # camera-to-world
    t = -R.T @ eye
    return R.astype(np.float32), t.astype(np.float32)
