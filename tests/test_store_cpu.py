"""Parameter store: fused Adam against torch.optim.Adam, record layouts, surgery."""
import torch

from retinags_b200.data import synthetic
from retinags_b200.models.gaussians import GaussianStore


def test_adam_matches_torch():
    g = synthetic.uniform_gaussians(37, 1, sh_degree=3)
    st = GaussianStore(37, "cpu")
    st.set_params(g)
    lrs = (1.6e-4, 2.5e-3, 2.5e-3 / 20, 5e-3, 1e-3, 5e-2)
    n = 37
    ref = {k: v.clone().requires_grad_(True) for k, v in g.items()}
    sh = ref["sh"].detach().view(n, 16, 3)
    f_dc = sh[:, :1].clone().requires_grad_(True)
    f_rest = sh[:, 1:].clone().requires_grad_(True)
    opt = torch.optim.Adam([
        {"params": [ref["xyz"]], "lr": lrs[0]}, {"params": [f_dc], "lr": lrs[1]}, {"params": [f_rest], "lr": lrs[2]},
        {"params": [ref["scale"]], "lr": lrs[3]}, {"params": [ref["rot"]], "lr": lrs[4]},
        {"params": [ref["opacity"]], "lr": lrs[5]}], lr=0.0, eps=1e-15)
    gen = torch.Generator().manual_seed(3)
    for _ in range(5):
        gv = st.views("grads")
        for name in ("xyz", "scale", "rot", "opacity"):
            gr = torch.randn(ref[name].shape, generator=gen) * 1e-3
            ref[name].grad = gr.clone()
            gv[name].copy_(gr)
        gr = torch.randn(n, 16, 3, generator=gen) * 1e-3
        f_dc.grad = gr[:, :1].clone()
        f_rest.grad = gr[:, 1:].clone()
        gv["sh"].copy_(gr.view(n, 48))
        opt.step()
        st.mark_touched()
        st.adam_step(lrs)
        assert float(st.grads.abs().sum()) == 0.0
    p = st.views()
    torch.testing.assert_close(p["xyz"], ref["xyz"].detach(), atol=5e-6, rtol=1e-5)
    torch.testing.assert_close(p["sh"].view(n, 16, 3)[:, :1], f_dc.detach(), atol=5e-6, rtol=1e-5)
    torch.testing.assert_close(p["sh"].view(n, 16, 3)[:, 1:], f_rest.detach(), atol=5e-6, rtol=1e-5)
    torch.testing.assert_close(p["opacity"], ref["opacity"].detach(), atol=5e-6, rtol=1e-5)
    torch.testing.assert_close(p["rot"], ref["rot"].detach(), atol=5e-6, rtol=1e-5)


def test_records_and_surgery():
    g = synthetic.uniform_gaussians(10, 2, sh_degree=3)
    st = GaussianStore(10, "cpu")
    st.set_params(g)
    rec = st.records()
    assert rec.shape == (10, 59)
    torch.testing.assert_close(rec[:, 0:3], g["xyz"])
    torch.testing.assert_close(rec[:, 3:51], g["sh"])
    torch.testing.assert_close(rec[:, 51:54], g["scale"])
    torch.testing.assert_close(rec[:, 54:58], g["rot"])
    torch.testing.assert_close(rec[:, 58:59], g["opacity"])
    st.exp_avg.normal_()
    mig = st.migration_records(torch.tensor([1, 4, 7]))
    assert mig.shape == (3, 177)
    other = GaussianStore(4, "cpu")
    other.append_migration(mig)
    assert other.count == 3
    torch.testing.assert_close(other.records(), rec[[1, 4, 7]])
    torch.testing.assert_close(other.records("exp_avg"), st.records("exp_avg")[[1, 4, 7]])
    keep = torch.ones(10, dtype=torch.bool)
    keep[[0, 5]] = False
    st.keep(keep)
    assert st.count == 8
    torch.testing.assert_close(st.records(), rec[keep])
    st.append_new({k: v[:2] for k, v in g.items()})
    assert st.count == 10 and st.cap >= 10
    torch.testing.assert_close(st.records()[8:], rec[:2])
    sd = st.optimizer_state_dict()
    st2 = GaussianStore(10, "cpu")
    st2.set_params({k: v for k, v in st.views().items()})
    st2.load_optimizer_state_dict(sd)
    torch.testing.assert_close(st2.records("exp_avg"), st.records("exp_avg"))


def test_untouched_rows_follow_dense_adam():
    """Rows without a gradient this step still decay their moments and move by momentum, exactly like dense Adam
    with a zero gradient; rows that never had a gradient are skipped and stay put."""
    g = synthetic.uniform_gaussians(12, 4, sh_degree=3)
    lrs = (1e-3,) * 6
    a, b = GaussianStore(12, "cpu"), GaussianStore(12, "cpu")
    a.set_params(g); b.set_params(g)
    gen = torch.Generator().manual_seed(0)
    rows = torch.tensor([0, 3, 7])
    for step in range(4):
        full = torch.randn(12, 59, generator=gen) * 1e-2
        if step >= 2:
            full[:] = 0  # later steps: nobody visible
        for st in (a, b):
            gv = st.views("grads")
            off = 0
            for name, w in zip(("xyz", "sh", "scale", "rot", "opacity"), (3, 48, 3, 4, 1)):
                gv[name][rows] = full[rows, off:off + w]
                off += w
        a.mark_touched()            # dense: every row is read
        if step < 2:
            b.mark_touched(rows)    # sparse bookkeeping: only rows that received a gradient
        a.adam_step(lrs); b.adam_step(lrs)
    torch.testing.assert_close(a.records(), b.records(), atol=0, rtol=0)
    torch.testing.assert_close(a.records("exp_avg"), b.records("exp_avg"), atol=0, rtol=0)
    untouched = torch.tensor([1, 2, 4, 5, 6, 8, 9, 10, 11])
    torch.testing.assert_close(b.records()[untouched], torch.cat([g[k] for k in ("xyz", "sh", "scale", "rot", "opacity")], 1)[untouched])


def _densify_store(n, device="cpu", seed=0):
    g = torch.Generator().manual_seed(seed)
    st = GaussianStore(n, device)
    st.set_params(dict(xyz=torch.randn(n, 3, generator=g), sh=torch.randn(n, 48, generator=g),
                       scale=torch.randn(n, 3, generator=g) * 0.7 - 2.0, rot=torch.randn(n, 4, generator=g),
                       opacity=torch.randn(n, 1, generator=g) * 2 - 1))
    st.exp_avg.copy_(torch.randn(st.exp_avg.shape, generator=g))
    st.exp_avg_sq.copy_(torch.rand(st.exp_avg_sq.shape, generator=g))
    st.grad_accum[:n] = (torch.rand(n, generator=g) * 0.001).to(st.device)
    st.denom[:n] = torch.randint(0, 4, (n,), generator=g).float().to(st.device)
    st.max_radii[:n] = (torch.rand(n, generator=g) * 40).to(st.device)
    return st


def test_native_densify_matches_torch_rules():
    """The classification/scan/compaction kernels (CPU twin) take the same decisions and produce the same row order as
    the PyTorch restatement; only the split offsets differ (another generator), and they have the right statistics."""
    from retinags_b200.models import densify
    from retinags_b200.models.gaussians import NAMES
    n = 5000
    cases = [dict(extent=5.0, max_screen_size=20.0), dict(extent=20.0, max_screen_size=None),
             dict(extent=20.0, max_screen_size=20.0, skip_clone=True), dict(extent=20.0, max_screen_size=20.0, skip_split=True),
             dict(extent=5.0, max_screen_size=None, skip_prune=True), dict(extent=5.0, max_screen_size=20.0, max_size=100)]
    saw_clone = saw_split = False
    for kw in cases:
        kw = dict(kw)
        extent = kw.pop("extent")
        a, b = _densify_store(n), _densify_store(n)
        parents = b.views()
        parent_xyz, parent_scale = parents["xyz"].clone(), parents["scale"].clone()
        densify.densify_and_prune(a, 0.0002, 0.005, extent, native_path=False, generator=torch.Generator().manual_seed(1), **kw)
        info = densify.densify_and_prune(b, 0.0002, 0.005, extent, native_path=True, seed=7, **kw)
        assert a.count == b.count
        k, sp = info["cloned"], info["split"]
        saw_clone |= k > 0
        saw_split |= sp > 0
        head = b.count - 2 * sp
        for which in ("params", "exp_avg", "exp_avg_sq"):
            va, vb = a.views(which), b.views(which)
            for nm in NAMES:
                if which == "params" and nm == "xyz":
                    assert torch.equal(va[nm][:head], vb[nm][:head])
                elif which == "params" and nm == "scale":
                    assert torch.allclose(va[nm], vb[nm], atol=1e-6)
                else:
                    assert torch.equal(va[nm], vb[nm]), (which, nm)
        assert float(b.grad_accum.abs().sum()) == 0 and float(b.grads.abs().sum()) == 0
        if sp > 200:
            # a child's offset, expressed in units of the parent's largest axis, is bounded and has zero mean
            child = b.views()["xyz"][head:]
            same = a.views()["xyz"][head:]
            assert not torch.allclose(child, same)
            spread = (child[:sp] - child[sp:]).norm(dim=1)  # the two children of one parent
            parent_max = torch.exp(b.views()["scale"][head:head + sp]).max(dim=1).values * 1.6
            ratio = spread / parent_max
            assert 0.3 < float(ratio.median()) < 2.5
    assert saw_clone and saw_split
    del parent_xyz, parent_scale


def test_native_densify_is_reproducible_and_seeded():
    from retinags_b200.models import densify
    a, b, c = _densify_store(3000), _densify_store(3000), _densify_store(3000)
    for st, seed in ((a, 5), (b, 5), (c, 6)):
        densify.densify_and_prune(st, 0.0002, 0.005, 5.0, 20.0, native_path=True, seed=seed)
    assert torch.equal(a.params, b.params)
    assert a.count == c.count and not torch.equal(a.params, c.params)


def test_split_samples_are_standard_normal():
    """Children of many identical unit Gaussians: offsets are N(0, I)."""
    from retinags_b200.models import densify
    n = 20000
    st = GaussianStore(n, "cpu")
    st.set_params(dict(xyz=torch.zeros(n, 3), sh=torch.zeros(n, 48), scale=torch.zeros(n, 3),
                       rot=torch.tensor([[1.0, 0, 0, 0]]).repeat(n, 1), opacity=torch.ones(n, 1)))
    st.grad_accum[:n] = 1.0
    st.denom[:n] = 1.0
    info = densify.densify_and_prune(st, 0.0002, 0.005, 1.0, None, native_path=True, seed=11)
    assert info["split"] == n and st.count == 2 * n
    x = st.views()["xyz"]
    assert abs(float(x.mean())) < 0.02 and abs(float(x.std()) - 1.0) < 0.02
    assert abs(float((x[:n] * x[n:]).mean())) < 0.02        # the two children are independent
    assert abs(float((x[:, 0] * x[:, 1]).mean())) < 0.02    # so are the axes
    assert abs(float((x ** 4).mean()) - 3.0) < 0.15          # kurtosis of a normal
    assert torch.allclose(st.views()["scale"], torch.full((2 * n, 3), -0.4700036), atol=1e-5)


def test_record_pack_matches_column_views():
    st = _densify_store(300)
    idx = torch.tensor([5, 0, 299, 17, 17])
    rec = st.migration_records(idx)
    want = torch.cat([st.records(w, idx) for w in ("params", "exp_avg", "exp_avg_sq")], dim=1)
    assert torch.equal(rec, want)
    assert torch.equal(st.migration_records(), torch.cat([st.records(w) for w in ("params", "exp_avg", "exp_avg_sq")], dim=1))
    other = GaussianStore(4, "cpu")
    other.append_migration(rec[:2])
    other.append_migration(rec[2:])
    assert other.count == 5 and torch.equal(other.migration_records(), rec)
