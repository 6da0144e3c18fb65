"""Dataset readers: COLMAP (binary and text), Blender/NeRF-synthetic transforms, ScanNet++ and Mill-19
style folders, plus the writer for the synthetic Blender-layout scenes used in benchmarks.

Behavioural parity: ``scene/dataset_readers.py:28-573`` and ``scene/colmap_loader.py:1-294`` of the
reference (camera conventions, the ``llffhold=8`` hold-out when ``--eval`` is given, the
"NeRF++" normalisation radius = 1.1 x the largest distance of a camera to the mean camera centre,
dataset type sniffing of ``scene/scene4bounded_gaussian.py:43-56``).  Images are *not* decoded here:
a ``CameraInfo`` only records the path; pixels are loaded lazily by the dataset
(``data/datasets.py``).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from ..models import ply_io
from ..utils import graphics


@dataclass
class CameraInfo:
    uid: int
    R: np.ndarray
    T: np.ndarray
    fovy: float
    fovx: float
    image_path: str
    image_name: str
    width: int
    height: int


@dataclass
class SceneInfo:
    points: np.ndarray | None
    colors: np.ndarray | None
    train_cameras: list
    test_cameras: list
    nerf_normalization: dict
    ply_path: str
    kind: str = ""


def nerfpp_norm(cam_infos: list[CameraInfo]) -> dict:
    centers = []
    for c in cam_infos:
        w2c = graphics.world_to_view(c.R, c.T)
        centers.append(np.linalg.inv(w2c.astype(np.float64))[:3, 3])
    centers = np.stack(centers, 0) if centers else np.zeros((1, 3))
    mean = centers.mean(0)
    radius = float(np.linalg.norm(centers - mean, axis=1).max()) * 1.1 if len(cam_infos) else 1.0
    return {"translate": -mean, "radius": radius}


# ---------------------------------------------------------------------------------------------
# COLMAP
# ---------------------------------------------------------------------------------------------
_CAMERA_MODELS = {0: ("SIMPLE_PINHOLE", 3), 1: ("PINHOLE", 4), 2: ("SIMPLE_RADIAL", 4), 3: ("RADIAL", 5), 4: ("OPENCV", 8),
                  5: ("OPENCV_FISHEYE", 8), 6: ("FULL_OPENCV", 12), 7: ("FOV", 5), 8: ("SIMPLE_RADIAL_FISHEYE", 4),
                  9: ("RADIAL_FISHEYE", 5), 10: ("THIN_PRISM_FISHEYE", 12)}
_MODEL_BY_NAME = {v[0]: (k, v[1]) for k, v in _CAMERA_MODELS.items()}


def qvec2rotmat(q) -> np.ndarray:
    w, x, y, z = q
    return np.array([[1 - 2 * y * y - 2 * z * z, 2 * x * y - 2 * w * z, 2 * z * x + 2 * w * y],
                     [2 * x * y + 2 * w * z, 1 - 2 * x * x - 2 * z * z, 2 * y * z - 2 * w * x],
                     [2 * z * x - 2 * w * y, 2 * y * z + 2 * w * x, 1 - 2 * x * x - 2 * y * y]])


def read_colmap_cameras(path: str) -> dict:
    cams = {}
    if path.endswith(".bin"):
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            for _ in range(n):
                cid, model, w, h = struct.unpack("<iiQQ", f.read(24))
                name, npar = _CAMERA_MODELS[model]
                params = struct.unpack("<" + "d" * npar, f.read(8 * npar))
                cams[cid] = dict(model=name, width=int(w), height=int(h), params=np.array(params))
    else:
        for line in open(path):
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            t = line.split()
            cams[int(t[0])] = dict(model=t[1], width=int(t[2]), height=int(t[3]), params=np.array([float(x) for x in t[4:]]))
    return cams


def read_colmap_images(path: str) -> dict:
    imgs = {}
    if path.endswith(".bin"):
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            for _ in range(n):
                iid = struct.unpack("<i", f.read(4))[0]
                q = struct.unpack("<dddd", f.read(32))
                t = struct.unpack("<ddd", f.read(24))
                cid = struct.unpack("<i", f.read(4))[0]
                name = b""
                while True:
                    ch = f.read(1)
                    if ch == b"\x00":
                        break
                    name += ch
                (npts,) = struct.unpack("<Q", f.read(8))
                f.seek(24 * npts, 1)
                imgs[iid] = dict(qvec=np.array(q), tvec=np.array(t), camera_id=cid, name=name.decode())
    else:
        lines = [ln.strip() for ln in open(path) if ln.strip() and not ln.startswith("#")]
        for ln in lines[0::2]:
            t = ln.split()
            imgs[int(t[0])] = dict(qvec=np.array([float(x) for x in t[1:5]]), tvec=np.array([float(x) for x in t[5:8]]),
                                   camera_id=int(t[8]), name=t[9])
    return imgs


def read_colmap_points(path: str):
    if path.endswith(".bin"):
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            xyz, rgb = np.empty((n, 3)), np.empty((n, 3))
            for i in range(n):
                rec = struct.unpack("<QdddBBBd", f.read(43))
                xyz[i], rgb[i] = rec[1:4], rec[4:7]
                (tl,) = struct.unpack("<Q", f.read(8))
                f.seek(8 * tl, 1)
        return xyz, rgb
    xyz, rgb = [], []
    for line in open(path):
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        t = line.split()
        xyz.append([float(x) for x in t[1:4]])
        rgb.append([int(x) for x in t[4:7]])
    return np.array(xyz), np.array(rgb)


def _colmap_cameras(src: str, images_dir: str) -> list[CameraInfo]:
    sp = os.path.join(src, "sparse", "0")
    if not os.path.isdir(sp):
        sp = os.path.join(src, "sparse")
    ext = ".bin" if os.path.exists(os.path.join(sp, "images.bin")) else ".txt"
    cams = read_colmap_cameras(os.path.join(sp, "cameras" + ext))
    imgs = read_colmap_images(os.path.join(sp, "images" + ext))
    out = []
    for k, (iid, im) in enumerate(sorted(imgs.items(), key=lambda kv: kv[1]["name"])):
        c = cams[im["camera_id"]]
        R = qvec2rotmat(im["qvec"]).T
        T = np.array(im["tvec"])
        if c["model"] in ("SIMPLE_PINHOLE", "SIMPLE_RADIAL"):
            fx = fy = c["params"][0]
        else:
            fx, fy = c["params"][0], c["params"][1]
        out.append(CameraInfo(uid=iid, R=R, T=T, fovy=graphics.focal2fov(fy, c["height"]),
                              fovx=graphics.focal2fov(fx, c["width"]),
                              image_path=os.path.join(src, images_dir, os.path.basename(im["name"])),
                              image_name=Path(im["name"]).stem, width=c["width"], height=c["height"]))
    return out


def _colmap_point_cloud(src: str, points3D: str, sample_rate: int):
    sp = os.path.join(src, "sparse", "0")
    if not os.path.isdir(sp):
        sp = os.path.join(src, "sparse")
    ply = os.path.join(sp, points3D + ".ply")
    if not os.path.exists(ply):
        binp, txtp = os.path.join(sp, points3D + ".bin"), os.path.join(sp, points3D + ".txt")
        xyz, rgb = read_colmap_points(binp if os.path.exists(binp) else txtp)
        ply_io.store_point_cloud(ply, xyz, rgb)
    pts, col, _ = ply_io.fetch_point_cloud(ply, sample_rate)
    return pts, col, ply


def read_colmap_scene(src: str, images: str = "images", eval_split: bool = False, points3D: str = "points3D",
                      sample_rate: int = 1, llffhold: int = 8) -> SceneInfo:
    cams = _colmap_cameras(src, images or "images")
    if eval_split:
        train = [c for i, c in enumerate(cams) if i % llffhold != 0]
        test = [c for i, c in enumerate(cams) if i % llffhold == 0]
    else:
        train, test = cams, []
    pts, col, ply = _colmap_point_cloud(src, points3D, sample_rate)
    return SceneInfo(pts, col, train, test, nerfpp_norm(train), ply, "Colmap")


def read_scannetpp_scene(src: str, points3D: str = "points3D", sample_rate: int = 1) -> SceneInfo:
    """COLMAP model + ``train_test_lists.json`` ({"train": [...], "test": [...]} image names)."""
    lists = json.load(open(os.path.join(src, "train_test_lists.json")))
    cams = _colmap_cameras(src, "images")
    tr = {Path(n).stem for n in lists.get("train", [])}
    te = {Path(n).stem for n in lists.get("test", [])}
    train = [c for c in cams if c.image_name in tr]
    test = [c for c in cams if c.image_name in te]
    pts, col, ply = _colmap_point_cloud(src, points3D, sample_rate)
    return SceneInfo(pts, col, train, test, nerfpp_norm(train), ply, "ScanNet++")


def read_mill19_scene(src: str, points3D: str = "points3D") -> SceneInfo:
    """COLMAP model whose test images live in ``test/`` and training images in ``train/`` (or ``images/``)."""
    cams = _colmap_cameras(src, "images")
    test_names = {Path(n).stem for n in os.listdir(os.path.join(src, "test"))} if os.path.isdir(os.path.join(src, "test")) else set()
    train, test = [], []
    for c in cams:
        if c.image_name in test_names:
            c.image_path = os.path.join(src, "test", os.path.basename(c.image_path))
            test.append(c)
        else:
            tp = os.path.join(src, "train", os.path.basename(c.image_path))
            if os.path.exists(tp):
                c.image_path = tp
            train.append(c)
    pts, col, ply = _colmap_point_cloud(src, points3D, 1)
    return SceneInfo(pts, col, train, test, nerfpp_norm(train), ply, "Mill19")


# ---------------------------------------------------------------------------------------------
# Blender / NeRF-synthetic
# ---------------------------------------------------------------------------------------------
def _blender_cameras(src: str, transforms: str, extension: str = "") -> list[CameraInfo]:
    path = os.path.join(src, transforms)
    if not os.path.exists(path):
        return []
    contents = json.load(open(path))
    out = []
    for idx, frame in enumerate(contents["frames"]):
        c2w = np.array(frame["transform_matrix"], dtype=np.float64)
        c2w[:3, 1:3] *= -1  # OpenGL (y up, z back) -> COLMAP (y down, z forward)
        w2c = np.linalg.inv(c2w)
        R, T = w2c[:3, :3].T, w2c[:3, 3]
        src_info = contents if "w" in contents else frame
        fovx, W, H = src_info["camera_angle_x"], int(src_info["w"]), int(src_info["h"])
        name = frame["file_path"] + extension
        if not os.path.splitext(name)[1] and os.path.exists(os.path.join(src, name + ".png")):
            name += ".png"
        out.append(CameraInfo(uid=idx, R=R, T=T, fovy=graphics.focal2fov(graphics.fov2focal(fovx, W), H), fovx=fovx,
                              image_path=os.path.join(src, name), image_name=Path(name).stem, width=W, height=H))
    return out


def read_blender_scene(src: str, eval_split: bool = False, points3D: str = "points3d", sample_rate: int = 1) -> SceneInfo:
    train = _blender_cameras(src, "transforms_train.json")
    test = _blender_cameras(src, "transforms_test.json")
    if not eval_split:
        train, test = train + test, []
    ply = os.path.join(src, points3D + ".ply")
    if not os.path.exists(ply):
        rng = np.random.default_rng(0)
        xyz = rng.random((100_000, 3)) * 2.6 - 1.3
        ply_io.store_point_cloud(ply, xyz, rng.random((100_000, 3)) * 255)
    pts, col, _ = ply_io.fetch_point_cloud(ply, sample_rate)
    return SceneInfo(pts, col, train, test, nerfpp_norm(train), ply, "Blender")


def read_scene(src: str, images: str = "images", eval_split: bool = False, points3D: str = "points3D",
               sample_rate: int = 1) -> SceneInfo:
    """Dataset type sniffing in the reference's order."""
    if os.path.exists(os.path.join(src, "sparse")):
        if os.path.exists(os.path.join(src, "train_test_lists.json")):
            return read_scannetpp_scene(src, points3D, sample_rate)
        if not os.path.exists(os.path.join(src, "test")):
            return read_colmap_scene(src, images, eval_split, points3D, sample_rate)
        return read_mill19_scene(src, points3D)
    if os.path.exists(os.path.join(src, "transforms_train.json")):
        return read_blender_scene(src, eval_split, points3D if points3D != "points3D" else "points3d", sample_rate)
    raise ValueError(f"could not recognise the scene type of {src}")


# ---------------------------------------------------------------------------------------------
# writer for synthetic scenes (Blender layout)
# ---------------------------------------------------------------------------------------------
def write_blender_scene(dst: str, train_cams, test_cams, points: np.ndarray | None = None, colors: np.ndarray | None = None):
    """Write cameras with their ``image`` tensors as PNG files plus ``transforms_{train,test}.json`` and an
    optional ``points3d.ply``; the result is readable by the reference and by :func:`read_scene`."""
    from ..utils.image import save_png

    os.makedirs(dst, exist_ok=True)
    for split, cams in (("train", train_cams), ("test", test_cams)):
        os.makedirs(os.path.join(dst, split), exist_ok=True)
        frames = []
        for cam in cams:
            w2c = np.eye(4)
            w2c[:3, :3] = np.asarray(cam.R, dtype=np.float64).T
            w2c[:3, 3] = np.asarray(cam.T, dtype=np.float64)
            c2w = np.linalg.inv(w2c)
            c2w[:3, 1:3] *= -1
            rel = f"{split}/{cam.image_name}.png"
            if cam.image is not None:
                save_png(os.path.join(dst, rel), cam.image)
            frames.append({"file_path": rel, "transform_matrix": c2w.tolist()})
        w, h = (cams[0].width, cams[0].height) if cams else (0, 0)
        fovx = cams[0].fovx if cams else 0.0
        json.dump({"camera_angle_x": fovx, "w": w, "h": h, "frames": frames},
                  open(os.path.join(dst, f"transforms_{split}.json"), "w"))
    if points is not None:
        col = colors if colors is not None else np.full_like(points, 128.0)
        ply_io.store_point_cloud(os.path.join(dst, "points3d.ply"), points, col)
