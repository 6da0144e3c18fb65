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
