"""Single-GPU scene holder with the interface of vanilla 3DGS (``Scene``).

Counterpart of the reference's legacy ``scene/scene.py:21-82`` / ``scene/simple_scene.py``: sniff the dataset type,
build the train/test camera lists, initialise a :class:`GaussianModel` from the point cloud or load
``<model>/point_cloud/iteration_N/point_cloud.ply``, write ``cameras.json`` and ``input.ply``, save per iteration.
The model-parallel trainer (``trainer.py``) has its own loader (``SceneV3`` in the reference); this class serves
single-GPU scripts and notebooks.
"""
from __future__ import annotations

import json
import os
import random
import shutil

from .data import readers
from .data.datasets import CameraListDataset
from .models.gaussian_model import GaussianModel


def search_for_max_iteration(folder: str) -> int:
    its = [int(name.split("_")[-1]) for name in os.listdir(folder) if name.startswith("iteration_")]
    return max(its)


class Scene:
    def __init__(self, args, gaussians: GaussianModel, load_iteration: int | None = None, shuffle: bool = True,
                 resolution_scales=(1.0,), scene_info: readers.SceneInfo | None = None):
        self.model_path = args.model_path
        self.gaussians = gaussians
        self.loaded_iter = None
        if load_iteration:
            pc_dir = os.path.join(self.model_path, "point_cloud")
            self.loaded_iter = search_for_max_iteration(pc_dir) if load_iteration == -1 else load_iteration
        info = scene_info if scene_info is not None else readers.read_scene(
            args.source_path, getattr(args, "images", "images"), getattr(args, "eval", False),
            getattr(args, "points3D", "points3D"), getattr(args, "pointcloud_sample_rate", 1))
        self.scene_info = info
        os.makedirs(self.model_path, exist_ok=True)
        if not self.loaded_iter:
            if info.ply_path and os.path.exists(info.ply_path):
                shutil.copyfile(info.ply_path, os.path.join(self.model_path, "input.ply"))
            cams = list(info.test_cameras) + list(info.train_cameras)
            with open(os.path.join(self.model_path, "cameras.json"), "w") as f:
                json.dump([_camera_json(i, c) for i, c in enumerate(cams)], f)
        train, test = list(info.train_cameras), list(info.test_cameras)
        if shuffle:
            rng = random.Random(0)
            rng.shuffle(train)
            rng.shuffle(test)
        self.cameras_extent = float(info.nerf_normalization["radius"])
        res, white = getattr(args, "resolution", -1), getattr(args, "white_background", False)
        self.train_cameras = {s: CameraListDataset(train, res, s, white) for s in resolution_scales}
        self.test_cameras = {s: CameraListDataset(test, res, s, white) for s in resolution_scales}
        if self.loaded_iter:
            self.gaussians.load_ply(os.path.join(self.model_path, "point_cloud", f"iteration_{self.loaded_iter}",
                                                 "point_cloud.ply"))
            self.gaussians.spatial_lr_scale = self.cameras_extent
        else:
            self.gaussians.create_from_pcd(info.points, info.colors, self.cameras_extent)

    def save(self, iteration: int):
        self.gaussians.save_ply(os.path.join(self.model_path, "point_cloud", f"iteration_{iteration}", "point_cloud.ply"))

    def getTrainCameras(self, scale: float = 1.0) -> CameraListDataset:
        return self.train_cameras[scale]

    def getTestCameras(self, scale: float = 1.0) -> CameraListDataset:
        return self.test_cameras[scale]


def _camera_json(idx: int, cam) -> dict:
    if hasattr(cam, "to_json"):
        return cam.to_json(idx)
    import numpy as np
    Rt = np.eye(4)
    Rt[:3, :3] = cam.R.T
    Rt[:3, 3] = cam.T
    c2w = np.linalg.inv(Rt)
    from .utils.graphics import fov2focal
    return dict(id=idx, img_name=cam.image_name, width=cam.width, height=cam.height, position=c2w[:3, 3].tolist(),
                rotation=[r.tolist() for r in c2w[:3, :3]], fy=fov2focal(cam.fovy, cam.height), fx=fov2focal(cam.fovx, cam.width))
