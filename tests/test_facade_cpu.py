"""Single-GPU facade (GaussianModel / Scene / render functions) and the headless viewer server, on CPU."""
import json
import os
import socket
import threading

import numpy as np
import torch

from retinags_b200.config import build_parser
from retinags_b200.data import readers, synthetic
from retinags_b200.gaussian_renderer import render, render_submodel
from retinags_b200.models.gaussian_model import GaussianModel
from retinags_b200.scene import Scene
from retinags_b200.viewer_server import ViewerServer


def _opt():
    parser, lp, op, pp = build_parser()
    args = parser.parse_args([])
    return op.extract(args)


def _targets(n_views=4, w=96, h=64):
    """Ground truth: renders of a reference model."""
    gt_model = GaussianModel(3, "cpu")
    g = synthetic.uniform_gaussians(1500, 7, sh_degree=3, log_scale_mean=-2.4)
    gt_model._replace_store(g)
    gt_model.active_sh_degree = 3
    cams = synthetic.ring_cameras(n_views, 3.0, w, h)
    for cam in cams:
        cam.image = gt_model.render(cam)["render"].clone()
    return gt_model, cams


def test_model_trains_saves_and_restores(tmp_path):
    gt_model, cams = _targets()
    pts = gt_model.get_xyz.numpy()
    cols = np.clip(gt_model.get_features[:, 0].numpy() * 0.28209479177387814 + 0.5, 0, 1)
    model = GaussianModel(3, "cpu")
    model.create_from_pcd(pts, cols, spatial_lr_scale=3.0)
    assert len(model) == 1500 and model.active_sh_degree == 0
    assert model.get_scaling.shape == (1500, 3) and torch.allclose(model.get_rotation.norm(dim=1), torch.ones(1500))
    assert torch.allclose(model.get_opacity, torch.full((1500, 1), 0.1), atol=1e-6)
    model.training_setup(_opt())
    losses = []
    for it in range(12):
        model.update_learning_rate(it)
        losses.append(model.train_step([cams[it % len(cams)]])["loss"])
    assert np.mean(losses[-4:]) < np.mean(losses[:4])
    model.oneupSHdegree()
    assert model.active_sh_degree == 1
    # files
    ply = str(tmp_path / "point_cloud" / "iteration_12" / "point_cloud.ply")
    model.save_ply(ply)
    other = GaussianModel(3, "cpu")
    other.load_ply(ply)
    torch.testing.assert_close(other.get_xyz, model.get_xyz)
    torch.testing.assert_close(other.get_features, model.get_features)
    # checkpoint with optimiser state
    state = model.capture()
    twin = GaussianModel(3, "cpu")
    twin.restore(state, _opt())
    assert twin.store.step == model.store.step
    torch.testing.assert_close(twin.store.records("exp_avg_sq"), model.store.records("exp_avg_sq"))
    a = model.train_step([cams[0]])["loss"]
    b = twin.train_step([cams[0]])["loss"]
    assert abs(a - b) < 1e-9
    # density control through the model interface
    n0 = len(model)
    info = model.densify_and_prune(1e-7, 0.005, 3.0, None, seed=3)
    assert len(model) == n0 + info["cloned"] + info["split"] - info["pruned"]
    model.reset_opacity()
    assert float(model.get_opacity.max()) <= 0.0100001
    out = model.render(cams[0])
    assert out["render"].shape == (3, 64, 96) and out["radii"].shape[0] == len(model)


def test_render_functions_agree():
    gt_model, cams = _targets(2)
    a = gt_model.render(cams[1], bg_color=(0.2, 0.3, 0.4))
    b = render(cams[1], gt_model, None, (0.2, 0.3, 0.4))
    torch.testing.assert_close(a["render"], b["render"], atol=1e-6, rtol=1e-5)
    assert torch.equal(a["visibility_filter"], b["visibility_filter"])
    # a bounded sub-model renders only what lies inside its box
    st = gt_model.store
    st.box_lo, st.box_hi = [-10.0, -10.0, -10.0], [0.0, 10.0, 10.0]
    half = render_submodel(cams[1], st, want_depth=True)
    assert half["depth"].shape == (1, 64, 96)
    assert float(half["alpha"].sum()) < float(b["alpha"].sum())
    st.box_lo, st.box_hi = [-np.inf] * 3, [np.inf] * 3


def test_scene_loads_blender_layout_and_saves(tmp_path):
    gt_model, cams = _targets(6)
    src = str(tmp_path / "scene")
    pts = gt_model.get_xyz.numpy()
    readers.write_blender_scene(src, cams[:5], cams[5:], pts, np.full_like(pts, 0.5))
    parser, lp, op, pp = build_parser()
    args = parser.parse_args(["-s", src, "-m", str(tmp_path / "model"), "--eval"])
    model = GaussianModel(3, "cpu")
    scene = Scene(lp.extract(args), model)
    assert len(scene.getTrainCameras()) == 5 and len(scene.getTestCameras()) == 1
    assert len(model) == pts.shape[0] and scene.cameras_extent > 0
    assert len(json.load(open(os.path.join(str(tmp_path / "model"), "cameras.json")))) == 6
    cam = scene.getTrainCameras()[0]
    assert cam.image.shape == (3, 64, 96)
    model.training_setup(op.extract(args))
    model.train_step([cam])
    scene.save(1)
    again = Scene(lp.extract(args), GaussianModel(3, "cpu"), load_iteration=-1)
    assert again.loaded_iter == 1 and len(again.gaussians) == len(model)


def test_viewer_server_answers_a_frame_request():
    gt_model, cams = _targets(1, 48, 32)
    server = ViewerServer("127.0.0.1", 0)
    cam = cams[0]
    wvt = cam.world_view_transform.copy().astype(np.float64)  # transposed world-to-view
    wvt[:, 1] *= -1
    wvt[:, 2] *= -1  # what an OpenGL viewer would send
    msg = dict(resolution_x=48, resolution_y=32, train=1, fov_y=cam.fovy, fov_x=cam.fovx, z_near=0.01, z_far=100.0,
               shs_python=0, rot_scale_python=0, keep_alive=1, scaling_modifier=1.0, view_matrix=wvt.reshape(-1).tolist(),
               view_projection_matrix=[0.0] * 16)
    reply = {}

    def viewer():
        with socket.create_connection((server.host, server.port), timeout=30) as s:
            raw = json.dumps(msg).encode()
            s.sendall(len(raw).to_bytes(4, "little") + raw)
            need = 48 * 32 * 3
            buf = b""
            while len(buf) < need + 4:
                buf += s.recv(65536)
            n = int.from_bytes(buf[need:need + 4], "little")
            while len(buf) < need + 4 + n:
                buf += s.recv(65536)
            reply["frame"], reply["path"] = buf[:need], buf[need + 4:need + 4 + n].decode()

    t = threading.Thread(target=viewer)
    t.start()
    req = None
    for _ in range(2000):
        req = server.serve_once(lambda c, s: gt_model.render(c)["render"], verify="/data/scene")
        if req is not None:
            break
        threading.Event().wait(0.005)
    t.join(30)
    server.close()
    assert req is not None and req.do_training and req.keep_alive
    assert reply["path"] == "/data/scene"
    frame = torch.frombuffer(bytearray(reply["frame"]), dtype=torch.uint8).view(32, 48, 3).permute(2, 0, 1).float() / 255
    want = cams[0].image.clamp(0, 1)
    assert float((frame - want).abs().max()) <= 1.0 / 255 + 1e-6
