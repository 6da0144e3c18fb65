"""Occlusion culling between sub-models (``StepEngine.render_partials_occluded``) on the CPU twins.

Four sub-models in one process (the maps are exchanged through the local transport) in a dense, opaque scene:
the culled training step must reproduce the step of a single model (which stops blending behind finished pixels by
itself) more closely than the step without culling does, with far fewer tile instances.
"""
import os

import torch

from retinags_b200.bench_session import BenchSession
from retinags_b200.ops import rasterize


def _session(occlusion: bool, depth: int, monkeypatch):
    monkeypatch.setenv("RGS_SLABS", "1")
    monkeypatch.setenv("RGS_SLAB_FRACTION", "64")
    monkeypatch.setattr(rasterize.RenderTask.__init__, "__defaults__", (4.0, 1 << 21, "depth_first"))  # no regrow in the test
    s = BenchSession("cpu", 0, 1, 30000, 160, 112, batch=2, n_views=4, gt_gaussians=5000, seed=5, sh_degree=1,
                     grid=(64, 64, 1), bvh_depth=depth, scene_kind="uniform")
    for st in s.stores.values():  # large opaque splats: most tiles are finished by the nearest sub-model
        v = st.views()
        v["opacity"] += 4.0
        v["scale"] += 1.2
    s.engine.occlusion = occlusion
    return s


def test_culled_step_matches_the_single_model_step(monkeypatch):
    single, plain, culled = _session(False, 0, monkeypatch), _session(False, 2, monkeypatch), _session(True, 2, monkeypatch)
    res = {}
    for name, s in (("single", single), ("plain", plain), ("culled", culled)):
        # no optimiser step: the gradients stay in the stores
        cams, rel = s._batch(0)
        r = s.engine.train_step(cams, rel, s.sh_degree, s.lrs, optimizer_step=False)
        info = s.engine.poll()
        assert not info["overflow"]
        img = torch.stack([s.engine._loss(v, 112, 160).image.clone() for v in range(2)])
        res[name] = dict(sums=torch.stack(r.sums), img=img, inst=info["n_inst"],
                         grad=torch.cat([st.records("grads") for _, st in sorted(s.stores.items())]),
                         xyz=torch.cat([st.xyz for _, st in sorted(s.stores.items())]))
    rel_err = lambda a, b: float(((a - b).abs() / b.abs().clamp_min(1e-12)).max())
    assert res["culled"]["inst"] * 2 < res["plain"]["inst"]
    e_culled, e_plain = rel_err(res["culled"]["sums"], res["single"]["sums"]), rel_err(res["plain"]["sums"], res["single"]["sums"])
    assert e_culled < 2e-5 and e_culled < e_plain
    assert float((res["culled"]["img"] - res["single"]["img"]).abs().max()) < 5e-4
    assert float((res["culled"]["img"] - res["plain"]["img"]).abs().max()) < 2e-2
    # same Gaussians, another order (grouped by sub-model): compare the gradients row by row after sorting by position
    def by_position(d):
        import numpy as np
        x = d["xyz"].numpy()
        return d["grad"][torch.from_numpy(np.lexsort((x[:, 2], x[:, 1], x[:, 0])))]
    gs, gc, gp = by_position(res["single"]), by_position(res["culled"]), by_position(res["plain"])
    assert float((gs - gc).norm()) <= 5e-4 * float(gs.norm())
    assert float((gs - gc).norm()) < float((gs - gp).norm())  # culling brings the split model closer to the single one


def test_culled_training_stays_close_to_the_plain_one(monkeypatch):
    plain, culled = _session(False, 2, monkeypatch), _session(True, 2, monkeypatch)
    la, lb = [], []
    for i in range(4):
        la.append(plain.step_e2e(i)[0])
        lb.append(culled.step_e2e(i)[0])
    assert culled.engine.dropped_steps == 0 and not culled.engine.poll()["overflow"]
    for x, y in zip(la, lb):
        assert abs(x - y) < 5e-3 * abs(x)
    assert lb[-1] < lb[0]


def test_border_sets_kept_for_eight_steps_train_like_sets_recomputed_every_step(monkeypatch):
    """``--BORROW_REFRESH_INTERVAL 8`` (selection kept, 5 % margin) against 1 (the reference's per-iteration selection)
    over 16 training steps of four sub-models: same losses, same parameters up to rounding."""
    monkeypatch.setenv("RGS_SLABS", "1")
    runs = {}
    for interval in (1, 8):
        s = BenchSession("cpu", 0, 1, 20000, 128, 96, batch=2, n_views=8, gt_gaussians=5000, seed=3, sh_degree=1,
                         grid=(64, 64, 1), bvh_depth=2, scene_kind="uniform", borrow_refresh=interval)
        for st in s.stores.values():
            st.views()["scale"] += 0.7  # more Gaussians reach over the borders
        assert int(s.border.refresh_interval) == interval
        losses = [s.step_e2e(i % 4)[0] for i in range(16)]
        runs[interval] = (losses, torch.cat([st.records() for _, st in sorted(s.stores.items())]),
                          int(s.border._counts.sum()))
    (l1, p1, n1), (l8, p8, n8) = runs[1], runs[8]
    assert n8 >= n1 > 0  # the kept sets are supersets (margin)
    for a, b in zip(l1, l8):
        assert abs(a - b) <= 1e-5 * abs(a)
    # Adam's steps have the size of the learning rate whatever the gradient's size, so rows whose gradient is rounding
    # noise may move differently (the lent rows arrive in another order, the sums round differently): few and small
    assert float((p1 - p8).abs().max()) < 2e-2 and float((p1 - p8).abs().mean()) < 1e-6
