"""End-to-end trainer on CPU: train from a point cloud with densification, checkpoint, resume, eval."""
import glob
import os

import numpy as np
import torch

from retinags_b200.config import build_parser
from retinags_b200.data.synthetic_scene import build_synthetic_scene
from retinags_b200.models import ply_io
from retinags_b200.trainer import Trainer


def _trainer(tmp, extra=(), scene=None):
    parser, lp, op, pp = build_parser()
    argv = ["-m", str(tmp), "--bvh_depth", "1", "--MAX_BATCH_SIZE", "2", "--MAX_LOAD", "4", "--device", "cpu",
            "--densify_from_iter", "4", "--densification_interval", "6", "--opacity_reset_interval", "1000",
            "--densify_until_iter", "40", "--quiet", "--EVAL_PSNR_INTERVAL", "2", "--eval"] + list(extra)
    args = parser.parse_args(argv)
    scene = scene or build_synthetic_scene("uniform:n=4000:w=96:h=64:views=10:test=2:init=1500:deg=1", device=torch.device("cpu"))
    return Trainer(args, lp.extract(args), op.extract(args), pp.extract(args), scene=scene), scene


def test_train_checkpoint_resume_eval(tmp_path):
    tr, scene = _trainer(tmp_path, ["--epochs", "3"])
    assert sorted(tr.stores) == [0, 1]
    n0 = sum(s.count for s in tr.stores.values())
    assert n0 == 1500
    before = tr.eval()
    tr.train()
    after = tr.eval()
    assert after["test"]["psnr"] > before["test"]["psnr"] + 0.5
    assert after["train"]["l1"] < before["train"]["l1"]
    n1 = sum(s.count for s in tr.stores.values())
    assert n1 != n0  # densification/pruning changed the point count
    it = tr.iteration
    ck = os.path.join(tmp_path, "rank_0", "point_cloud", f"iteration_{it}")
    assert os.path.exists(os.path.join(ck, "point_cloud_0.ply")) and os.path.exists(os.path.join(ck, "adam_1.pt"))
    assert os.path.exists(os.path.join(ck, "tree_0.txt"))
    whole = os.path.join(tmp_path, "point_cloud", f"iteration_{it}", "point_cloud.ply")
    g = ply_io.load_gaussians(whole)
    assert g["xyz"].shape[0] == n1
    names = ply_io.read_ply_vertices(whole).dtype.names
    assert list(names[:9]) == ["x", "y", "z", "nx", "ny", "nz", "f_dc_0", "f_dc_1", "f_dc_2"] and len(names) == 62
    # resume from the merged model with a different partition depth (whole-model mode)
    tr2, _ = _trainer(tmp_path, ["--epochs", "3", "--bvh_depth", "2"], scene)
    assert tr2.iteration == it and sum(s.count for s in tr2.stores.values()) == n1 and tr2.n_models == 4
    r2 = tr2.eval()
    assert abs(r2["test"]["psnr"] - after["test"]["psnr"]) < 0.3
    # resume from the per-sub-model files, Adam moments included
    tr3, _ = _trainer(tmp_path, ["--epochs", "4", "--SPLIT_MODEL"], scene)
    assert tr3.iteration == it and {m: s.count for m, s in tr3.stores.items()} == {m: s.count for m, s in tr.stores.items()}
    assert float(tr3.stores[0].exp_avg_sq.abs().sum()) > 0
    tr.stores[0].spatial_sort()  # the loader keeps the rows in Morton order of their current positions
    torch.testing.assert_close(tr3.stores[0].records("exp_avg"), tr.stores[0].records("exp_avg"))
    tr3.train()
    assert tr3.iteration > it


def test_repartition_keeps_every_gaussian(tmp_path):
    tr, _ = _trainer(tmp_path, ["--epochs", "1"])
    n = sum(s.count for s in tr.stores.values())
    for st in tr.stores.values():
        st.exp_avg.uniform_()
    rec_before = torch.cat([s.migration_records() for s in tr.stores.values()])
    # move everything so that the old partition is unbalanced, then rebalance
    for st in tr.stores.values():
        st.views()["xyz"][:, 0] += 0.35
    rec_before = torch.cat([s.migration_records() for s in tr.stores.values()])
    tr._repartition()
    assert sum(s.count for s in tr.stores.values()) == n
    rec_after = torch.cat([s.migration_records() for s in tr.stores.values()])
    a = rec_before[torch.argsort(rec_before[:, 0])]
    b = rec_after[torch.argsort(rec_after[:, 0])]
    torch.testing.assert_close(a, b)
    lo, hi = tr.boxes
    for m, st in tr.stores.items():
        p = st.xyz
        assert bool(((p > torch.tensor(lo[m], dtype=torch.float32)) & (p <= torch.tensor(hi[m], dtype=torch.float32))).all())
    counts = [s.count for s in tr.stores.values()]
    assert min(counts) > 0.6 * max(counts)


def test_anomaly_check_names_the_submodel_and_debug_mode_polls():
    """--detect_anomaly / pipe.debug: a NaN parameter is reported with sub-model and group; debug mode checks status words."""
    import pytest
    from retinags_b200.bench_session import BenchSession
    sess = BenchSession("cpu", 0, 1, 4000, 96, 64, batch=1, n_views=2, gt_gaussians=2000, seed=1, sh_degree=1, grid=(32, 32, 1),
                        bvh_depth=1, scene_kind="uniform")
    eng = sess.engine
    eng.debug = True
    eng.detect_anomaly = True
    sess.step(0)  # a healthy step passes both checks
    # the rasteriser itself is robust against NaN parameters (such Gaussians are culled); a NaN target is not survivable
    sess.cams[1].image[:, 10:20, 10:20] = float("nan")
    with pytest.raises(FloatingPointError) as err:
        sess.step(1)
    assert "non-finite loss sums" in str(err.value)
    victim = sorted(sess.stores)[1]
    st = sess.stores[victim]
    for other in sess.stores.values():
        other.zero_grad()  # the failed step left its NaN gradients behind
    st.views("grads")["scale"][3, 1] = float("inf")
    with pytest.raises(FloatingPointError) as err:
        eng._anomaly_check([])
    assert f"sub-model {victim}" in str(err.value) and "'scale'" in str(err.value) and "Gaussian 3" in str(err.value)


def test_whole_model_is_streamed_in_chunks_and_not_share_keeps_reaching_gaussians(tmp_path, monkeypatch):
    """The whole-model loader walks the file in chunks (here 300 rows) and ends with the same sub-models as labelling
    everything at once; with --NOT_SHRAE_GS_INFO a sub-model also keeps the Gaussians of its neighbours whose 3-sigma
    extent reaches into its box (nothing is borrowed later), and only those."""
    g = {k: v for k, v in __import__("retinags_b200.data.synthetic", fromlist=["x"]).uniform_gaussians(2500, 7, sh_degree=3).items()}
    it = 40
    os.makedirs(tmp_path / "point_cloud" / f"iteration_{it}")
    whole = str(tmp_path / "point_cloud" / f"iteration_{it}" / "point_cloud.ply")
    ply_io.save_gaussians(whole, g, 3, chunk=700)
    assert ply_io.PlyVertexStream(whole).count == 2500
    torch.testing.assert_close(ply_io.load_gaussians(whole)["sh"], g["sh"])
    monkeypatch.setattr(Trainer, "LOAD_CHUNK_ROWS", 300)
    tr, scene = _trainer(tmp_path, ["--epochs", "1", "--bvh_depth", "2"])
    assert tr.iteration == it and tr.n_models == 4 and sum(s.count for s in tr.stores.values()) == 2500
    ids = tr.tree.label(g["xyz"])
    for m, st in tr.stores.items():
        want = g["xyz"][ids == m]
        torch.testing.assert_close(st.xyz[torch.argsort(st.xyz[:, 0])], want[torch.argsort(want[:, 0])])
    assert tr.border is not None
    tr2, _ = _trainer(tmp_path, ["--epochs", "1", "--bvh_depth", "2", "--NOT_SHRAE_GS_INFO"], scene)
    assert tr2.border is None
    lo, hi = tr2.boxes
    r = 3.0 * torch.exp(g["scale"]).max(dim=1, keepdim=True).values
    total = 0
    for m, st in tr2.stores.items():
        reach = ((g["xyz"] + r >= torch.tensor(lo[m], dtype=torch.float32)) &
                 (g["xyz"] - r <= torch.tensor(hi[m], dtype=torch.float32))).all(dim=1)
        assert st.count == int(reach.sum()) and st.count >= int((ids == m).sum())
        total += st.count
    assert total > 2500  # border Gaussians live in more than one sub-model
    # the merge concatenates bytes and equals the parts in order
    parts = [str(tmp_path / f"part_{k}.ply") for k in range(2)]
    ply_io.save_gaussians(parts[0], {k: v[:1000] for k, v in g.items()}, 3)
    ply_io.save_gaussians(parts[1], {k: v[1000:] for k, v in g.items()}, 3)
    assert ply_io.merge_gaussian_files(str(tmp_path / "merged.ply"), parts, 3, block_rows=256) == 2500
    assert open(tmp_path / "merged.ply", "rb").read() == open(whole, "rb").read()
