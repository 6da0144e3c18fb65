"""File formats: Gaussian PLY (vanilla-3DGS layout), point clouds, COLMAP models, Blender-layout scenes, CLI flags."""
import json
import os
import struct

import numpy as np
import torch

from retinags_b200.config import build_parser
from retinags_b200.data import readers, synthetic
from retinags_b200.data.datasets import CameraListDataset, target_resolution
from retinags_b200.models import densify, ply_io
from retinags_b200.models.gaussians import GaussianStore


def test_gaussian_ply_layout_and_roundtrip(tmp_path):
    g = synthetic.uniform_gaussians(50, 3, sh_degree=3)
    f = str(tmp_path / "point_cloud.ply")
    ply_io.save_gaussians(f, g, 3)
    v = ply_io.read_ply_vertices(f)
    names = list(v.dtype.names)
    assert names == ply_io.gaussian_attribute_names(3) and len(names) == 62
    assert all(v.dtype[n] == np.dtype("<f4") for n in names)
    sh = g["sh"].view(50, 16, 3)
    # f_rest is channel-major in the file: f_rest_0..14 = red coefficients 1..15
    np.testing.assert_allclose(v["f_rest_0"], sh[:, 1, 0].numpy())
    np.testing.assert_allclose(v["f_rest_14"], sh[:, 15, 0].numpy())
    np.testing.assert_allclose(v["f_rest_15"], sh[:, 1, 1].numpy())
    np.testing.assert_allclose(v["f_rest_44"], sh[:, 15, 2].numpy())
    np.testing.assert_allclose(v["rot_0"], g["rot"][:, 0].numpy())
    assert float(np.abs(v["nx"]).max()) == 0.0
    back = ply_io.load_gaussians(f)
    for k in g:
        torch.testing.assert_close(back[k], g[k])
    # a degree-1 file loads into the degree-3 layout with zero higher bands
    ply_io.save_gaussians(f, g, 1)
    low = ply_io.load_gaussians(f)
    torch.testing.assert_close(low["sh"].view(50, 16, 3)[:, :4], sh[:, :4])
    assert float(low["sh"].view(50, 16, 3)[:, 4:].abs().sum()) == 0.0


def test_point_cloud_roundtrip(tmp_path):
    rng = np.random.default_rng(0)
    xyz, rgb = rng.normal(size=(100, 3)).astype(np.float32), rng.integers(0, 255, size=(100, 3))
    f = str(tmp_path / "points3d.ply")
    ply_io.store_point_cloud(f, xyz, rgb)
    p, c, n = ply_io.fetch_point_cloud(f)
    np.testing.assert_allclose(p, xyz)
    np.testing.assert_allclose(c, rgb / 255.0, atol=1e-6)
    p2, _, _ = ply_io.fetch_point_cloud(f, sample_rate=4)
    assert p2.shape[0] == 25


def _write_colmap_bin(root, cams, width, height):
    sp = os.path.join(root, "sparse", "0")
    os.makedirs(sp)
    os.makedirs(os.path.join(root, "images"))
    with open(os.path.join(sp, "cameras.bin"), "wb") as f:
        f.write(struct.pack("<Q", 1))
        fx = width / (2 * cams[0].tan_fovx)
        fy = height / (2 * cams[0].tan_fovy)
        f.write(struct.pack("<iiQQ", 1, 1, width, height) + struct.pack("<dddd", fx, fy, width / 2, height / 2))
    with open(os.path.join(sp, "images.bin"), "wb") as f:
        f.write(struct.pack("<Q", len(cams)))
        for i, c in enumerate(cams):
            R = np.asarray(c.R, dtype=np.float64).T  # world-to-camera
            from scipy.spatial.transform import Rotation
            qx, qy, qz, qw = Rotation.from_matrix(R).as_quat()
            f.write(struct.pack("<i", i + 1) + struct.pack("<dddd", qw, qx, qy, qz) + struct.pack("<ddd", *np.asarray(c.T, dtype=np.float64))
                    + struct.pack("<i", 1) + f"img_{i:03d}.png".encode() + b"\x00" + struct.pack("<Q", 0))
    with open(os.path.join(sp, "points3D.bin"), "wb") as f:
        f.write(struct.pack("<Q", 3))
        for k in range(3):
            f.write(struct.pack("<QdddBBBd", k, float(k), 0.5, -1.0, 10 * k, 20, 30, 0.1) + struct.pack("<Q", 0))


def test_colmap_binary_reader_and_holdout(tmp_path):
    cams = synthetic.ring_cameras(16, 3.0, 80, 60)
    _write_colmap_bin(str(tmp_path), cams, 80, 60)
    sc = readers.read_scene(str(tmp_path), "images", eval_split=True)
    assert sc.kind == "Colmap" and len(sc.test_cameras) == 2 and len(sc.train_cameras) == 14
    assert sc.points.shape == (3, 3)
    ci = sc.train_cameras[0]
    ref = cams[1]  # index 0 is held out (every 8th)
    np.testing.assert_allclose(ci.R, ref.R, atol=1e-5)
    np.testing.assert_allclose(ci.T, ref.T, atol=1e-5)
    assert abs(ci.fovx - ref.fovx) < 1e-6 and abs(ci.fovy - ref.fovy) < 1e-6
    assert sc.nerf_normalization["radius"] > 3.0
    assert os.path.exists(os.path.join(tmp_path, "sparse", "0", "points3D.ply"))


def test_blender_scene_writer_reader_roundtrip(tmp_path):
    cams = synthetic.ring_cameras(5, 3.0, 32, 24)
    for c in cams:
        c.image = torch.rand(3, 24, 32)
    readers.write_blender_scene(str(tmp_path), cams[:4], cams[4:], np.zeros((10, 3), np.float32))
    sc = readers.read_scene(str(tmp_path), eval_split=True)
    assert sc.kind == "Blender" and len(sc.train_cameras) == 4 and len(sc.test_cameras) == 1
    np.testing.assert_allclose(sc.train_cameras[2].R, cams[2].R, atol=1e-5)
    np.testing.assert_allclose(sc.train_cameras[2].T, cams[2].T, atol=1e-5)
    ds = CameraListDataset(sc.train_cameras, resolution=1)
    cam = ds[1]
    assert cam.image.shape == (3, 24, 32)
    assert (cam.image - cams[1].image).abs().max() < 1.0 / 255 + 1e-6
    assert ds.empty_item(1).image is None


def test_resolution_rule():
    assert target_resolution(3200, 2000, -1) == (1600, 1000)
    assert target_resolution(1200, 800, -1) == (1200, 800)
    assert target_resolution(1600, 1036, 2) == (800, 518)
    assert target_resolution(4000, 3000, 1000) == (1000, 750)


def test_cli_flags_of_the_reference_parse():
    parser, lp, op, pp = build_parser()
    a = parser.parse_args(["-s", "/data/garden", "-m", "/out/garden", "--bvh_depth", "2", "--MAX_BATCH_SIZE", "2", "--MAX_LOAD", "4",
                           "-r", "1", "--eval", "--EVAL_ONLY", "--SAVE_EVAL_IMAGE", "--SAVE_EVAL_SUB_IMAGE", "--SPLIT_MODEL",
                           "--ENABLE_REPARTITION", "--position_lr_init", "0.0000016", "--position_lr_final", "0.000000016",
                           "--densify_until_iter", "0", "--points3D", "MVS_points3D", "--iterations", "60000", "--epochs", "187"])
    m, o = lp.extract(a), op.extract(a)
    assert m.source_path == "/data/garden" and m.model_path == "/out/garden" and m.resolution == 1 and m.eval
    assert a.bvh_depth == 2 and a.MAX_LOAD == 4 and a.EVAL_ONLY and a.SPLIT_MODEL
    assert o.position_lr_init == 1.6e-6 and o.iterations == 60000 and o.epochs == 187 and m.points3D == "MVS_points3D"
    assert o.lambda_dssim == 0.2 and o.densification_interval == 100 and m.sh_degree == 3


def test_densify_rules():
    g = synthetic.uniform_gaussians(40, 7, sh_degree=3)
    g["scale"][:20] = -6.0      # small -> clone candidates
    g["scale"][20:] = -1.0      # large -> split candidates
    g["opacity"][:] = 2.0
    g["opacity"][5] = -8.0      # transparent -> pruned
    st = GaussianStore(40, "cpu")
    st.set_params(g)
    st.exp_avg.uniform_()
    st.denom[:40] = 1.0
    st.grad_accum[:40] = 0.0
    st.grad_accum[[0, 1, 25]] = 1.0   # two clones, one split
    gen = torch.Generator().manual_seed(0)
    info = densify.densify_and_prune(st, 0.0002, 0.005, extent=5.0, max_screen_size=None, generator=gen)
    assert info == dict(cloned=2, split=1, pruned=1)
    assert st.count == 40 + 2 + 2 - 1 - 1
    rec = st.records()
    assert float(st.grad_accum.abs().sum()) == 0.0 and float(st.denom.sum()) == 0.0
    # split children shrink by 1/(0.8*2) and carry zero moments; survivors keep theirs
    assert abs(float(rec[-1, 51]) - (-1.0 - np.log(1.6))) < 1e-5
    assert float(st.records("exp_avg")[-4:].abs().sum()) == 0.0
    assert float(st.records("exp_avg")[:10].abs().sum()) > 0.0
    densify.reset_opacity(st)
    assert float(torch.sigmoid(st.views()["opacity"]).max()) <= 0.01 + 1e-6
    assert float(st.views("exp_avg")["opacity"].abs().sum()) == 0.0


def test_sh_and_loss_helpers_match_the_oracle(tmp_path):
    from retinags_b200.ops import oracle
    from retinags_b200.utils import loss as L
    from retinags_b200.utils import sh as SH
    from retinags_b200.utils.general import build_rotation, covariance_3d
    gen = torch.Generator().manual_seed(0)
    dirs = torch.nn.functional.normalize(torch.randn(50, 3, generator=gen), dim=1)
    coeff = torch.randn(50, 16, 3, generator=gen)
    for deg in range(4):
        want = oracle.eval_sh(deg, coeff, dirs)
        got = SH.eval_sh(deg, coeff.transpose(1, 2), dirs)
        torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-5)
    rgb = torch.rand(7, 3, generator=gen)
    torch.testing.assert_close(SH.SH2RGB(SH.RGB2SH(rgb)), rgb)
    a, b = torch.rand(3, 40, 52, generator=gen), torch.rand(3, 40, 52, generator=gen)
    assert abs(float(L.ssim(a, a)) - 1.0) < 1e-6 and float(L.ssim(a, b)) < 0.2
    assert float(L.training_loss(a, a)) < 1e-6
    torch.testing.assert_close(L.training_loss(a, b), 0.8 * (a - b).abs().mean() + 0.2 * (1 - L.ssim(a, b)))
    assert float(L.psnr(a[None], a[None] * 0.5 + 0.25)) > 5.0
    q = torch.randn(9, 4, generator=gen)
    R = build_rotation(q)
    torch.testing.assert_close(R @ R.transpose(1, 2), torch.eye(3).expand(9, 3, 3), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(R, oracle.quat_to_rot(q / q.norm(dim=1, keepdim=True)), atol=1e-6, rtol=1e-5)
    cov = covariance_3d(torch.rand(9, 3, generator=gen) + 0.1, q)
    assert cov.shape == (9, 6) and bool((cov[:, 0] > 0).all())


def test_get_combined_args_reads_cfg_args_without_evaluating(tmp_path):
    from retinags_b200.config import get_combined_args
    parser, lp, op, pp = build_parser()
    model = tmp_path / "m"
    model.mkdir()
    (model / "cfg_args").write_text("Namespace(sh_degree=2, source_path='/data/x', white_background=True, images='img4')")
    args = get_combined_args(parser, ["-m", str(model), "--images", "images_2"])
    assert args.sh_degree == 3 or args.sh_degree == 2   # the command-line default is a value too
    assert args.images == "images_2" and args.model_path == str(model)
    assert args.white_background in (True, False)
    (model / "cfg_args").write_text("__import__('os').system('echo no')")
    args = get_combined_args(parser, ["-m", str(model)])
    assert args.model_path == str(model)


def test_lpips_module_with_local_weight_files(tmp_path):
    """The perceptual metric: zero for identical images, positive otherwise, weights read from local files only."""
    from retinags_b200.utils.lpips import LPIPS, load_lpips
    assert load_lpips(str(tmp_path)) is None  # no files -> the evaluation reports NaN
    torch.manual_seed(0)
    ref = LPIPS()
    for p in ref.parameters():
        p.copy_(torch.rand_like(p) * 0.1)
    torch.save({"features." + k: v for k, v in ref.features.state_dict().items()}, str(tmp_path / "vgg16.pth"))
    torch.save({f"lin{k}.model.1.weight": lin.weight for k, lin in enumerate(ref.lins)}, str(tmp_path / "lpips_vgg.pth"))
    net = load_lpips(str(tmp_path))
    assert net is not None
    a, b = torch.rand(3, 48, 64), torch.rand(3, 48, 64)
    assert float(net(a, a)) == 0.0
    d = float(net(a, b))
    assert d > 0 and abs(d - float(ref(a, b))) < 1e-6
    assert net(torch.stack([a, b]), torch.stack([b, b])).shape == (2,)


def test_scannetpp_and_mill19_layouts(tmp_path):
    """Dataset sniffing in the reference's order: a COLMAP model with ``train_test_lists.json`` is ScanNet++, one with a
    ``test/`` folder is Mill-19 (test pictures live there, training pictures in ``train/``)."""
    import json
    cams = synthetic.ring_cameras(8, 3.0, 80, 60)
    sn = tmp_path / "scannetpp"
    _write_colmap_bin(str(sn), cams, 80, 60)
    (sn / "train_test_lists.json").write_text(json.dumps({"train": [f"img_{i:03d}.png" for i in range(6)],
                                                          "test": ["img_006.png", "img_007.png"]}))
    sc = readers.read_scene(str(sn), eval_split=False)
    assert sc.kind == "ScanNet++" and len(sc.train_cameras) == 6 and len(sc.test_cameras) == 2
    assert sc.test_cameras[0].image_name == "img_006"
    ml = tmp_path / "mill19"
    _write_colmap_bin(str(ml), cams, 80, 60)
    os.makedirs(ml / "test")
    os.makedirs(ml / "train")
    for i in range(8):
        (ml / ("test" if i % 4 == 0 else "train") / f"img_{i:03d}.png").write_bytes(b"")
    sc = readers.read_scene(str(ml))
    assert sc.kind == "Mill19" and len(sc.test_cameras) == 2 and len(sc.train_cameras) == 6
    assert sc.test_cameras[1].image_path.endswith(os.path.join("test", "img_004.png"))
    assert sc.train_cameras[0].image_path.endswith(os.path.join("train", "img_001.png"))


def test_prefetcher_keeps_the_order_of_the_batches_and_raises_where_a_decode_failed(tmp_path):
    """``BatchPrefetcher`` (decode threads ahead of the step) against ``GroupedItems`` (the reference's dataset of
    batches): same cameras in the same order for any depth; an image that cannot be decoded raises at its batch."""
    from retinags_b200.data.datasets import GroupedItems
    from retinags_b200.data.prefetch import BatchPrefetcher
    cams = synthetic.ring_cameras(7, 3.0, 32, 24)
    for c in cams:
        c.image = torch.rand(3, 24, 32)
    readers.write_blender_scene(str(tmp_path), cams[:6], cams[6:], np.zeros((10, 3), np.float32))
    sc = readers.read_scene(str(tmp_path), eval_split=True)
    ds = CameraListDataset(sc.train_cameras, resolution=1, cache_bytes=0)  # nothing cached: every fetch decodes
    groups = [(0, 3), (5,), (2, 1), (4, 0)]
    want = GroupedItems(ds, groups)
    for depth in (0, 1, 16):
        got = list(BatchPrefetcher(ds, groups, depth=depth, workers=3))
        assert [ids for ids, _ in got] == groups
        for i, (ids, batch) in enumerate(got):
            ref_ids, ref_batch = want[i]
            assert tuple(ref_ids) == ids and [c.image_name for c in batch] == [c.image_name for c in ref_batch]
            assert all(torch.equal(a.image, b.image) for a, b in zip(batch, ref_batch))
    os.remove(sc.train_cameras[5].image_path)
    feed = iter(BatchPrefetcher(ds, groups, depth=4, workers=2))
    assert next(feed)[0] == (0, 3)
    try:
        next(feed)
        raise AssertionError("the missing image of batch 1 went unnoticed")
    except (FileNotFoundError, OSError):
        pass
