"""sm_100a kernels against the native CPU backend / PyTorch references (needs a B200)."""
import os

import pytest
import torch

from helpers import assert_mostly_close, native_render, small_scene
from retinags_b200.data import synthetic
from retinags_b200.models.gaussians import GaussianStore
from retinags_b200.ops import native, rasterize
from retinags_b200.ops.loss import CompositeLoss

pytestmark = pytest.mark.gpu


def _scene(n=40000, w=320, h=208, deg=3, seed=4):
    g = synthetic.uniform_gaussians(n, seed, sh_degree=deg, log_scale_mean=-3.6)
    cams = synthetic.ring_cameras(3, 3.0, w, h)
    return g, cams


def test_cuda_library_is_loaded():
    lib = native.lib("cuda")
    assert hasattr(lib, "rgs_cuda_blend_fwd")


@pytest.mark.parametrize("deg,box", [(3, (None, None)), (1, ([-0.2, -1e9, -1e9], [1e9, 0.3, 1e9]))])
def test_raster_forward_matches_cpu(deg, box):
    g, cams = _scene(deg=deg)
    for cam in cams[:2]:
        ref, tr, _, _ = native_render(g, cam, deg, box=box, device="cpu", want_depth=True)
        out, tg, _, _ = native_render(g, cam, deg, box=box, device="cuda", want_depth=True)
        assert tg.n_vis == tr.n_vis and tg.n_inst == tr.n_inst
        assert_mostly_close(out.cpu(), ref, atol=3e-5, rtol=1e-4)
        assert_mostly_close(tg.depth.cpu(), tr.depth, atol=2e-4, rtol=1e-4, hard_atol=5e-2)
        assert (tg.n_contrib.cpu() != tr.n_contrib).float().mean() < 1e-3


def test_binning_variants_agree_on_gpu():
    g, cams = _scene(n=60000)
    for cam in cams[:2]:
        a, ta, _, _ = native_render(g, cam, 3, device="cuda", binning="depth_first")
        b, tb, _, _ = native_render(g, cam, 3, device="cuda", binning="keyed")
        assert ta.n_vis == tb.n_vis and ta.n_inst <= tb.n_inst
        # splats of exactly equal depth are ordered by slot number, which differs between the pipelines
        assert_mostly_close(a, b, atol=1e-5, rtol=1e-4, max_frac=1e-2)
        ref, tr, _, _ = native_render(g, cam, 3, device="cpu", binning="depth_first")
        assert tr.n_inst == ta.n_inst
        assert_mostly_close(a.cpu(), ref, atol=3e-5, rtol=1e-4, max_frac=5e-3)


def test_tile_culling_is_exact_on_gpu():
    g, cams = _scene(n=60000)
    seg = rasterize.Segment(*(g[k].cuda().contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
    outs, insts = [], []
    for mode in (1, 2):
        task = rasterize.RenderTask("cuda")
        task.slabs = False  # the per-tile test replaces the two-slab forward: compare the two single-pass variants
        out = task.forward(rasterize.make_camera(cams[1], 3, tight_rect=mode), [seg], check=True)
        outs.append(out.clone()); insts.append(task.n_inst)
    assert torch.equal(outs[0], outs[1])
    assert insts[1] < insts[0]


def test_raster_small_capacity_regrows():
    g, cams = _scene(n=20000)
    seg = rasterize.Segment(*(g[k].cuda().contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
    task = rasterize.RenderTask("cuda", inst_per_gaussian=0.01, min_inst=256)
    c = rasterize.make_camera(cams[0], 3)
    out = task.forward(c, [seg], check=True)
    ref, _, _, _ = native_render(g, cams[0], 3, device="cpu")
    assert_mostly_close(out.cpu(), ref, atol=3e-5, rtol=1e-4)


@pytest.mark.parametrize("holes", [False, True])
def test_raster_backward_matches_cpu(holes):
    """``holes``: the incoming gradient is exactly zero on most of the image (pixels, 8x4 strips and whole tiles), which
    the CUDA blend backward skips and the CPU loops walk through."""
    deg = 3
    g, cams = _scene(n=20000, w=160, h=112)
    cam = cams[1]
    gen = torch.Generator().manual_seed(0)
    grad = torch.randn(cam.height, cam.width, 4, generator=gen)
    if holes:
        grad[:64] = 0.0
        grad[64:, ::3] = 0.0
        grad[80:100, 48:120] = 0.0
    res = {}
    for dev in ("cpu", "cuda"):
        out, task, seg, c = native_render(g, cam, deg, device=dev)
        n = seg.count
        for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1), ("g_mean2d", 2)):
            setattr(seg, name, torch.zeros(n, w, device=dev))
        seg.stat_grad = torch.zeros(n, device=dev)
        seg.stat_denom = torch.zeros(n, device=dev)
        seg.stat_maxrad = torch.zeros(n, device=dev)
        task.backward(grad.to(dev).contiguous(), [seg])
        res[dev] = seg
    for name in ("g_xyz", "g_sh", "g_scale", "g_rot", "g_opacity", "g_mean2d", "stat_grad", "stat_denom", "stat_maxrad"):
        a, b = getattr(res["cuda"], name).cpu(), getattr(res["cpu"], name)
        # atomics reorder the sums and a stop-rule flip changes single pixels: compare in norm
        assert (a - b).norm().item() <= 5e-3 * b.norm().item() + 1e-9, name


def test_radix_sort_matches_torch():
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda").manual_seed(1)
    for n, tiles in ((1, 7), (4097, 1000), (1_000_003, 6500), (3_000_000, 70000)):
        tile = torch.randint(0, tiles, (n,), device=dev, generator=gen, dtype=torch.int64)
        depth = torch.rand(n, device=dev, generator=gen) * 10 + 0.2
        keys = (tile << 32) | depth.view(torch.int32).to(torch.int64)
        vals = torch.arange(n, device=dev, dtype=torch.int32)
        cap = n + 123
        kbuf = torch.zeros(cap, dtype=torch.int64, device=dev); kbuf[:n] = keys
        vbuf = torch.zeros(cap, dtype=torch.int32, device=dev); vbuf[:n] = vals
        counters = torch.zeros(native.CNT_WORDS, dtype=torch.int32, device=dev)
        counters[native.CNT_INST] = n
        sc = rasterize.sort_scratch(dev)
        sc.ensure(cap)
        ranges = torch.zeros(tiles, 2, dtype=torch.int32, device=dev)
        native.call("sort_ranges", dev, kbuf, vbuf, sc.keys_tmp, sc.vals_tmp, cap, counters, tiles, ranges, sc.words)
        order = torch.sort(keys, stable=True).indices.to(torch.int32)
        assert torch.equal(vbuf[:n], order)
        sorted_tiles = tile[order.long()]
        counts = torch.bincount(sorted_tiles, minlength=tiles)
        ends = torch.cumsum(counts, 0)
        starts = ends - counts
        nz = counts > 0
        assert torch.equal(ranges[nz, 0].long(), starts[nz]) and torch.equal(ranges[nz, 1].long(), ends[nz])
        assert int(ranges[~nz].abs().sum()) == 0


def test_loss_kernels_match_cpu():
    H, W, K = 200, 333, 3
    gen = torch.Generator().manual_seed(0)
    parts = []
    for _ in range(K):
        T = torch.rand(H, W, 1, generator=gen) * 0.9 + 0.05
        parts.append(torch.cat([torch.rand(H, W, 3, generator=gen) * (1 - T), T], -1).contiguous())
    gt = torch.rand(3, H, W, generator=gen)
    bg = (0.1, 0.0, 0.3)
    res = {}
    for dev in ("cpu", "cuda"):
        cl = CompositeLoss(dev, H, W)
        p = [x.to(dev) for x in parts]
        cl.composite(p, bg)
        sums = cl.loss(gt.to(dev), 0.2).cpu()
        grads = [torch.zeros_like(x) for x in p]
        cl.backward(p, grads, bg)
        res[dev] = (cl.image.cpu(), sums, cl.g_image.cpu(), [x.cpu() for x in grads])
    torch.testing.assert_close(res["cuda"][0], res["cpu"][0], atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(res["cuda"][1], res["cpu"][1], atol=1e-2, rtol=1e-5)
    torch.testing.assert_close(res["cuda"][2], res["cpu"][2], atol=1e-9, rtol=2e-3)
    for a, b in zip(res["cuda"][3], res["cpu"][3]):
        torch.testing.assert_close(a, b, atol=1e-9, rtol=2e-3)


def test_adam_matches_cpu():
    g = synthetic.uniform_gaussians(1001, 1, sh_degree=3)
    lrs = (1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2)
    stores = {}
    for dev in ("cpu", "cuda"):
        st = GaussianStore(1001, dev)
        st.set_params({k: v.to(dev) for k, v in g.items()})
        gen = torch.Generator().manual_seed(3)
        for _ in range(3):
            full = (torch.randn(st.grads.shape, generator=gen) * 1e-3).to(dev)
            for name, view in st.views("grads").items():  # live rows only; padding rows stay untouched
                view.copy_(dict(GaussianStore._views(full, st.cap, st.count))[name])
            st.mark_touched(torch.arange(0, st.count, 2, device=dev))  # odd rows: their gradient must be ignored
            ref_rows = torch.arange(1, st.count, 2, device=dev)
            for view in st.views("grads").values():
                view[ref_rows] = 0
            st.adam_step(lrs)
        stores[dev] = st
    torch.testing.assert_close(stores["cuda"].records().cpu(), stores["cpu"].records(), atol=2e-6, rtol=1e-5)
    torch.testing.assert_close(stores["cuda"].records("exp_avg_sq").cpu(), stores["cpu"].records("exp_avg_sq"),
                               atol=1e-12, rtol=1e-5)
    assert float(stores["cuda"].grads.abs().sum()) == 0.0


def test_adam_row_block_variant_matches_unit_variant():
    """Both work distributions of the fused Adam give the same bits: sparse marks, dense marks, a tail that is not a
    multiple of 32 rows."""
    g = synthetic.uniform_gaussians(1001, 1, sh_degree=3)
    lrs = (1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2)
    stores = {}
    for variant in ("units", "rows"):
        st = GaussianStore(1001, "cuda")
        st.adam_variant = variant
        st.set_params({k: v.cuda() for k, v in g.items()})
        gen = torch.Generator().manual_seed(3)
        for step in range(4):
            full = (torch.randn(st.grads.shape, generator=gen) * 1e-3).cuda()
            for name, view in st.views("grads").items():
                view.copy_(dict(GaussianStore._views(full, st.cap, st.count))[name])
            rows = torch.arange(0, st.count, 7 if step < 2 else 1, device="cuda")  # sparse steps, then dense ones
            keep = torch.zeros(st.count, dtype=torch.bool, device="cuda")
            keep[rows] = True
            for view in st.views("grads").values():
                view[~keep] = 0
            st.mark_touched(rows)
            st.adam_step(lrs)
        stores[variant] = st
    for which in ("params", "exp_avg", "exp_avg_sq", "grads"):
        assert torch.equal(getattr(stores["units"], which), getattr(stores["rows"], which)), which
    assert torch.equal(stores["units"].active, stores["rows"].active)


def test_peer_transport_single_rank_equals_local():
    """The fused push path (blend epilogue stores into compositing slots, flag signal/wait kernels, gradient
    images inside the exchange region) with world size 1 must reproduce the local transport."""
    from retinags_b200.bench_session import BenchSession
    from retinags_b200.parallel.peer import PeerTransport

    def make():
        return BenchSession("cuda", 0, 1, 60000, 320, 208, batch=2, n_views=4, gt_gaussians=20000, seed=5, sh_degree=3,
                            grid=(64, 64, 1), bvh_depth=1)
    a, b = make(), make()
    from retinags_b200.parallel.peer_border import PeerBorderExchange
    tr = PeerTransport(torch.device("cuda"))
    b.engine.transport = tr
    lo, hi = b.tree.leaf_boxes_world(open_border=True)
    b.engine.borrow = PeerBorderExchange(lo, hi, b.model2rank, 0, 1, torch.device("cuda"), tr, None, refresh_interval=1)
    ia, _, _ = a.render_view(1)
    ib, _, _ = b.render_view(1)
    torch.testing.assert_close(ia, ib, atol=1e-6, rtol=1e-5)
    for i in range(2):
        la = a.step_e2e(i)[0]
        lb = b.step_e2e(i)[0]
        assert abs(la - lb) < 1e-4 * max(1.0, abs(la))
    torch.cuda.synchronize()
    tr.check()
    assert int(b.engine.borrow._counts.sum()) == int(a.border._counts.sum()) > 0
    for m in a.stores:
        ra, rb = a.stores[m].records(), b.stores[m].records()
        assert (ra - rb).abs().mean() < 1e-5
    b.engine.borrow.close()
    tr.close()


def test_ssim_tensor_core_path_matches_simt():
    """tcgen05/TMEM horizontal filter (3xTF32) against the fp32 SIMT statistics kernel."""
    from retinags_b200.ops import loss as loss_mod
    H, W = 300, 448
    gen = torch.Generator().manual_seed(3)
    img = torch.rand(3, H, W, generator=gen).cuda()
    gt = (img.cpu() + 0.1 * torch.randn(3, H, W, generator=gen)).clamp(0, 1).cuda()
    res = {}
    for tc in (False, True):
        cl = CompositeLoss("cuda", H, W)
        cl.tensor_cores = tc and cl._tc_supported()
        if tc:
            assert cl.tensor_cores, "tensor-core SSIM path not available"
        cl.image.copy_(img)
        sums = cl.loss(gt, 0.2, 16, 280).clone()
        torch.cuda.synchronize()
        assert int(cl.status[0]) == 0, f"bounded wait expired in the tensor-core kernel (status {int(cl.status[0])})"
        res[tc] = (sums.cpu(), cl.dmaps[:, 11:285].clone().cpu(), cl.g_image[:, 16:280].clone().cpu())
    torch.testing.assert_close(res[True][0], res[False][0], atol=1e-2, rtol=2e-5)
    d_ref = res[False][1]
    assert (res[True][1] - d_ref).abs().max().item() <= 2e-3 * d_ref.abs().max().item()
    g_ref = res[False][2]
    assert (res[True][2] - g_ref).abs().max().item() <= 2e-3 * g_ref.abs().max().item()


def test_aux_kernels_match_cpu():
    """kNN initialiser, load histogram and frustum mask on the GPU against their CPU twins."""
    from retinags_b200.ops.knn import knn3_dist2
    from retinags_b200.parallel.partition import Grid3D, load_histogram
    gen = torch.Generator().manual_seed(0)
    pts = torch.cat([torch.randn(40000, 3, generator=gen), torch.rand(200, 3, generator=gen) * 30])
    torch.testing.assert_close(knn3_dist2(pts.cuda()).cpu(), knn3_dist2(pts), atol=1e-9, rtol=1e-5)
    grid = Grid3D.from_points(pts.numpy().astype("float64"), (64, 32, 1))
    torch.testing.assert_close(load_histogram(pts.cuda(), grid).cpu(), load_histogram(pts, grid))


def test_surgery_kernels_match_cpu():
    """Densification (classify, scan, compaction with Philox split samples) and migration records: GPU against the CPU twin."""
    from retinags_b200.models import densify
    from test_store_cpu import _densify_store
    for n, kw in ((7000, dict(extent=5.0, max_screen_size=20.0)), (2500, dict(extent=20.0, max_screen_size=None))):
        extent = kw.pop("extent")
        a, b = _densify_store(n, "cpu"), _densify_store(n, "cuda")
        ia = densify.densify_and_prune(a, 0.0002, 0.005, extent, native_path=True, seed=9, **kw)
        ib = densify.densify_and_prune(b, 0.0002, 0.005, extent, native_path=True, seed=9, **kw)
        assert ia == ib and a.count == b.count
        for which in ("params", "exp_avg", "exp_avg_sq"):
            va, vb = a.views(which), b.views(which)
            for nm in va:
                torch.testing.assert_close(vb[nm].cpu(), va[nm], atol=2e-5, rtol=1e-5)
        idx = torch.randperm(a.count)[:333]
        torch.testing.assert_close(b.migration_records(idx.cuda()).cpu(), a.migration_records(idx), atol=2e-5, rtol=1e-5)
        c = GaussianStore(8, "cuda")
        c.append_migration(b.migration_records())
        assert torch.equal(c.migration_records(), b.migration_records())


@pytest.mark.parametrize("K", [3, 10])
def test_fused_composite_loss_matches_separate_kernels(K):
    """The two fused training kernels against the four separate ones on the GPU, and against the CPU twin; up to 8
    partials the backward kernels keep the prefix products in registers, above that in a local array."""
    g = torch.Generator().manual_seed(5)
    H, W = 150, 203
    parts = [torch.cat([torch.rand(H, W, 3, generator=g) * 0.4, torch.rand(H, W, 1, generator=g)], dim=2).contiguous()
             for _ in range(K)]
    gt = torch.rand(3, H, W, generator=g)
    bg = (0.1, 0.2, 0.3)
    for rows in ((0, H), (37, 101)):
        out = {}
        for dev, fused in (("cuda", False), ("cuda", True), ("cpu", True)):
            cl = CompositeLoss(dev, H, W)
            pp = [p.to(dev) for p in parts]
            gg = [torch.zeros(H, W, 4, device=dev) for _ in range(K)]
            if fused:
                s = cl.fused_loss_backward(pp, gg, gt.to(dev), bg, 0.2, rows[0], rows[1]).clone()
            else:
                cl.composite(pp, bg, max(0, rows[0] - 10), min(H, rows[1] + 10))
                s = cl.loss(gt.to(dev), 0.2, rows[0], rows[1]).clone()
                cl.backward(pp, gg, bg, rows[0], rows[1])
            out[(dev, fused)] = (s.cpu(), [x.cpu() for x in gg], cl.image[:, rows[0]:rows[1]].cpu())
        # the same fused kernels as 2 x 2 thread-block clusters: the same arithmetic per pixel, hence the same bits
        was = native.cuda_switch("loss_cluster", True)
        try:
            cl = CompositeLoss("cuda", H, W)
            gg = [torch.zeros(H, W, 4, device="cuda") for _ in range(K)]
            s = cl.fused_loss_backward([p.cuda() for p in parts], gg, gt.cuda(), bg, 0.2, rows[0], rows[1]).clone()
        finally:
            native.cuda_switch("loss_cluster", was)
        plain = out[("cuda", True)]
        torch.testing.assert_close(s.cpu(), plain[0], rtol=1e-12, atol=0)  # double sums, other order of the atomics
        assert torch.equal(cl.image[:, rows[0]:rows[1]].cpu(), plain[2])
        assert all(torch.equal(x.cpu(), y) for x, y in zip(gg, plain[1]))
        ref = out[("cuda", False)]
        for key in (("cuda", True), ("cpu", True)):
            got = out[key]
            torch.testing.assert_close(got[0], ref[0], rtol=5e-5, atol=1e-6)  # fp32 partial sums in another order
            torch.testing.assert_close(got[2], ref[2], rtol=1e-6, atol=1e-7)
            for x, y in zip(got[1], ref[1]):
                torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-9)


def test_segmented_counting_grouping_matches_radix(tmp_path):
    """The optional tile grouping without a second sort (RGS_TILE_GROUPING=count, read once per process) renders the same
    image as the radix grouping, with both rectangle modes."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, torch\n"
        f"sys.path.insert(0, {os.path.join(root, 'tests')!r}); sys.path.insert(0, {root!r})\n"
        "from retinags_b200.data import synthetic\n"
        "from retinags_b200.ops import rasterize\n"
        "g = synthetic.uniform_gaussians(60000, 4, sh_degree=3, log_scale_mean=-3.6)\n"
        "cams = synthetic.ring_cameras(3, 3.0, 320, 208)\n"
        "seg = rasterize.Segment(*(g[k].cuda().contiguous() for k in ('xyz', 'sh', 'scale', 'rot', 'opacity')))\n"
        "outs = []\n"
        "for mode in (1, 2):\n"
        "    task = rasterize.RenderTask('cuda')\n"
        "    outs.append((task.forward(rasterize.make_camera(cams[1], 3, tight_rect=mode), [seg], check=True).cpu(), task.n_inst))\n"
        "torch.save(outs, sys.argv[1])\n")
    res = {}
    for mode in ("radix", "count"):
        path = str(tmp_path / f"{mode}.pt")
        env = dict(os.environ, RGS_TILE_GROUPING=mode)
        proc = subprocess.run([sys.executable, "-c", code, path], env=env, capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
        res[mode] = torch.load(path)
    for (a, na), (b, nb) in zip(res["radix"], res["count"]):
        assert na == nb
        assert torch.equal(a, b)


def test_deterministic_backward_mode_gives_identical_bits():
    """Fixed-point accumulation in the blend backward: two backward passes over the same forward agree bit for bit (the
    float-atomic path generally does not) and stay close to the float-atomic result."""
    g, cams = _scene(n=30000, w=240, h=160)
    cam = cams[1]
    grad = torch.randn(cam.height, cam.width, 4, generator=torch.Generator().manual_seed(1)).cuda().contiguous()
    out, task, seg, c = native_render(g, cam, 3, device="cuda")
    n = seg.count
    runs = []
    for deterministic in (True, True, False):
        task.deterministic = deterministic
        task.splat_grads.zero_()  # the projection zeroes them once per forward; a second backward starts from zero again
        for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1)):
            setattr(seg, name, torch.zeros(n, w, device="cuda"))
        task.backward(grad, [seg])
        task._record_counters()  # status word after the backward (index guards, bounded waits)
        torch.cuda.synchronize()
        assert task.poll()["status"] == 0
        runs.append(torch.cat([seg.g_xyz, seg.g_sh, seg.g_scale, seg.g_rot, seg.g_opacity], dim=1).cpu())
    assert torch.equal(runs[0], runs[1])
    assert (runs[0] - runs[2]).norm().item() <= 1e-4 * runs[2].norm().item()
    assert float(runs[0].abs().sum()) > 0


def test_peer_region_canaries_detect_an_out_of_bounds_store():
    """The guard zones around an exchange region: intact after normal use, flagged after a store one byte past the end
    (the store stays inside the allocation, nothing faults)."""
    from retinags_b200.parallel.peer import GUARD_BYTES, PeerRegion
    region = PeerRegion(4096, torch.device("cuda", 0))
    region.view(0, (1024,)).fill_(3.0)
    region.view(4096 - 16, (4,)).fill_(7.0)
    assert region.verify_canaries()
    region._whole[GUARD_BYTES + region.nbytes] = 1  # what an off-by-one peer store would hit
    assert not region.verify_canaries()
    region.close()


def test_two_slab_forward_matches_single_pass_and_emits_fewer_instances():
    """Near slab first, far slab only for unsaturated tiles: same image, contributor indices and gradients as the single
    pass, fewer tile instances in a dense opaque scene."""
    g = synthetic.uniform_gaussians(150000, 5, sh_degree=3, log_scale_mean=-3.0)
    g["opacity"] = g["opacity"] + 4.0
    cams = synthetic.ring_cameras(3, 3.0, 320, 208)
    grad = torch.randn(208, 320, 4, generator=torch.Generator().manual_seed(2)).cuda().contiguous()
    res = {}
    for slabs in (False, True):
        seg = rasterize.Segment(*(g[k].cuda().contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
        task = rasterize.RenderTask("cuda")
        task.slabs = slabs
        task.deterministic = True
        out = task.forward(rasterize.make_camera(cams[1], 3), [seg], want_depth=True, check=True).clone()
        n = seg.count
        for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1)):
            setattr(seg, name, torch.zeros(n, w, device="cuda"))
        task.backward(grad, [seg])
        task._record_counters()
        torch.cuda.synchronize()
        assert task.poll()["status"] == 0
        res[slabs] = (out, task.n_contrib.clone(), task.depth.clone(), task.n_inst,
                      torch.cat([seg.g_xyz, seg.g_sh, seg.g_scale, seg.g_rot, seg.g_opacity], dim=1))
    a, b = res[False], res[True]
    assert (a[0][..., 3] < 1e-3).float().mean() > 0.3, "the scene does not saturate"
    # two renders number their slots independently, and splats of exactly equal depth are ordered by slot number: single
    # pixels may differ in the last bits, everything else is identical
    assert_mostly_close(a[0], b[0], atol=1e-5, rtol=1e-4, max_frac=1e-2)
    assert (a[1] != b[1]).float().mean() < 1e-2, f"contributor index differs at {int((a[1] != b[1]).sum())} pixels"
    assert_mostly_close(a[2], b[2], atol=2e-4, rtol=1e-4, max_frac=1e-2, hard_atol=5e-2)
    assert b[3] < a[3], f"instances: single pass {a[3]}, two slabs {b[3]}"
    assert (a[4] - b[4]).norm().item() <= 1e-3 * a[4].norm().item(), "gradients differ"


def test_cuda_render_and_gradients_match_the_pytorch_oracle():
    """The CUDA path against the independent fp32 PyTorch restatement (``ops/oracle.py``), not against the CPU build of
    the same header: forward image, transmittance and depth, and all five parameter gradients through autograd."""
    from helpers import activated
    from retinags_b200.ops import oracle
    deg = 3
    g, cams = small_scene(n=500, seed=21, width=96, height=64)
    cam = cams[1]
    box = ([-0.4, -1e9, -1e9], [1e9, 0.5, 1e9])
    a = activated(g)
    leaves = {k: v.clone().requires_grad_(True) for k, v in a.items()}
    C, T, D, _ = oracle.rasterize(cam, leaves["xyz"], leaves["sh"].view(-1, 16, 3), leaves["opacity"], leaves["scale"],
                                  leaves["rot"], deg, box[0], box[1])
    gen = torch.Generator().manual_seed(0)
    wC, wT, wD = torch.randn(C.shape, generator=gen), torch.randn(T.shape, generator=gen), torch.randn(D.shape, generator=gen)
    ((C * wC).sum() + (T * wT).sum() + (D * wD).sum()).backward()
    out, task, seg, c = native_render(a, cam, deg, box=box, raw=False, device="cuda", want_depth=True)
    ref = torch.cat([C.detach().permute(1, 2, 0), T.detach()[..., None]], dim=-1)
    assert (out.cpu() - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())
    assert (task.depth.cpu() - D.detach()).abs().max().item() <= 1e-4 * max(1.0, D.abs().max().item())
    n = seg.count
    for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1)):
        setattr(seg, name, torch.zeros(n, w, device="cuda"))
    grad = torch.cat([wC.permute(1, 2, 0), wT[..., None]], dim=-1).contiguous().cuda()
    task.backward(grad, [seg], grad_depth=wD.contiguous().cuda())
    for name, key in (("g_xyz", "xyz"), ("g_sh", "sh"), ("g_scale", "scale"), ("g_rot", "rot"), ("g_opacity", "opacity")):
        want = leaves[key].grad
        got = getattr(seg, name).cpu()
        assert (got - want).norm().item() <= 2e-3 * want.norm().item() + 1e-9, name


def test_a_device_wait_that_runs_out_reports_and_leaves_the_context_usable():
    """Failure detection on the device without a fault: a wait on an epoch that nobody will signal gives up after its
    cycle budget, records which rank it waited for, the kernel returns normally and the host check raises. Afterwards
    the same transport signals and waits as usual."""
    from retinags_b200.parallel.peer import PeerTransport
    dev = torch.device("cuda", 0)
    tr = PeerTransport(dev)
    tr._local_index = {0: 0}
    tr._ensure(4096, 4096, 1, 1, 1)
    tr.barrier()
    torch.cuda.synchronize()
    tr.check()  # healthy
    native.call("p2p_wait", dev, tr.flags, 1, tr.epoch + 3, 2_000_000, tr.status, None, sig="piiippp")  # ~1 ms budget
    torch.cuda.synchronize()
    assert int(tr.status[0]) == 0x100
    tr.record_status()
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="peer wait expired: no signal from rank 0"):
        tr.check(block=False)
    with pytest.raises(RuntimeError, match="peer wait expired"):
        tr.check()
    tr.status.zero_()
    tr.barrier()
    torch.cuda.synchronize()
    tr.check()
    assert float(torch.ones(4, device=dev).sum()) == 4.0
    tr.close()


def test_border_selection_kernel_matches_the_mask_selection_on_gpu():
    """``rgs_border_mask_kernel`` (one pass, bit mask per Gaussian) against the boolean-mask selection, four boxes."""
    from retinags_b200.parallel.border import select_border
    g = synthetic.uniform_gaussians(50000, 9, sh_degree=1, log_scale_mean=-3.0)
    st = GaussianStore(50000, "cuda", 1)
    st.set_params({k: v.cuda() for k, v in g.items()})
    lo = torch.tensor([[-9., -9, -9], [0, -9, -9], [-9, 0, -9], [0, 0, -9]]).cuda()
    hi = torch.tensor([[0., 0, 9], [9, 0, 9], [0, 9, 9], [9, 9, 9]]).cuda()
    for m in range(4):
        a = select_border(st, m, lo, hi, 0.05, native_mask=False)
        b = select_border(st, m, lo, hi, 0.05, native_mask=True)
        assert sorted(a) == sorted(b) and len(a) > 0
        for d in a:
            assert torch.equal(a[d], b[d])


def test_an_overflowing_step_is_dropped_by_the_optimiser_and_leaves_no_gradients():
    """A render that runs out of instance capacity raises the overflow word; the fused Adam sees it, changes no
    parameter, clears the step's gradients, and the next step (buffers grown by the poll) trains normally."""
    from retinags_b200.bench_session import BenchSession
    sess = BenchSession("cuda", 0, 1, 60000, 320, 208, batch=2, n_views=4, gt_gaussians=20000, seed=5, sh_degree=3,
                        grid=(64, 64, 1), bvh_depth=1)
    sess.step(0); sess.settle()
    for task in sess.engine._tasks.values():  # shrink every instance buffer far below the need
        task._grow_inst(task.min_inst)
        task.cap_inst = 4096
        task._pending_cap = 0
    before = [st.params.clone() for st in sess.stores.values()]
    sess.step(1)
    torch.cuda.synchronize()
    assert int(sess.engine._skip[native.CNT_OVERFLOW]) != 0
    for st, b in zip(sess.stores.values(), before):
        assert torch.equal(st.params, b)
        assert float(st.grads.abs().sum()) == 0.0 and int(st.touched.sum()) == 0
    info = None
    while info is None:
        info = sess.engine.poll_async()
    assert info["dropped"] and info["overflow"]
    sess.step(2)
    torch.cuda.synchronize()
    assert int(sess.engine._skip[native.CNT_OVERFLOW]) == 0
    assert any(not torch.equal(st.params, b) for st, b in zip(sess.stores.values(), before))


def test_single_sweep_sort_orders_like_the_three_kernel_sort():
    """Binning with the look-back scatter against the histogram / scan / scatter passes. Two renders number their slots
    in the order of the projection's atomics, so the sorted lists are checked for what the blend relies on (tile by
    tile, depth ascending, equal depths by slot) and the images are compared, not the slot numbers. 400 k splats give
    the depth sort about a hundred chunks and the tile sort several hundred, more than one per SM."""
    g, cams = _scene(n=400000)
    was = native.cuda_switch("sort_sweep", True)
    try:
        for cam in cams[:2]:
            for slabs in (True, False):
                got = {}
                for sweep in (True, False):
                    native.cuda_switch("sort_sweep", sweep)
                    seg = rasterize.Segment(*(g[k].cuda().contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
                    task = rasterize.RenderTask("cuda")
                    task.slabs = slabs
                    img = task.forward(rasterize.make_camera(cam, 3), [seg], check=True).clone()
                    got[sweep] = (img, task.n_vis, task.n_inst, task.ranges.clone())
                    if not slabs:
                        vals = task.vals[:task.n_inst].long()
                        depth = rasterize.bin_scratch(torch.device("cuda")).slot_depth.view(torch.int32)[vals]
                        starts = task.ranges[:, 0][task.ranges[:, 1] > task.ranges[:, 0]].long()
                        inside = torch.ones(task.n_inst - 1, dtype=torch.bool, device="cuda")
                        inside[starts[starts > 0] - 1] = False  # pairs that straddle two tiles
                        assert not ((depth[1:] < depth[:-1]) & inside).any(), "depth order broken inside a tile"
                        assert not ((depth[1:] == depth[:-1]) & (vals[1:] < vals[:-1]) & inside).any(), "not stable"
                        assert int((task.ranges[:, 1] - task.ranges[:, 0]).sum()) == task.n_inst
                assert got[True][1:3] == got[False][1:3]
                assert torch.equal(got[True][3], got[False][3])
                assert_mostly_close(got[True][0], got[False][0], atol=1e-5, rtol=1e-4, max_frac=1e-3)
    finally:
        native.cuda_switch("sort_sweep", was)


def test_two_slab_forward_with_more_than_65536_tiles():
    """A 4400 x 4000 image has 68 750 tiles: the tile keys of the slabs need a third 8-bit pass (and the single-sweep
    sort ends in the other buffer); the image equals the single-pass render."""
    g = synthetic.uniform_gaussians(60000, 6, sh_degree=1, log_scale_mean=-3.2)
    cam = synthetic.ring_cameras(3, 3.0, 4400, 4000)[1]
    assert (4400 + 15) // 16 * ((4000 + 15) // 16) > 65536
    out = {}
    for slabs in (False, True):
        seg = rasterize.Segment(*(g[k].cuda().contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
        task = rasterize.RenderTask("cuda")
        task.slabs = slabs
        out[slabs] = task.forward(rasterize.make_camera(cam, 1), [seg], check=True).clone()
        assert task._slab_active == slabs
        del task
    assert float(out[False][..., :3].sum()) > 0
    assert_mostly_close(out[False], out[True], atol=1e-5, rtol=1e-4, max_frac=1e-2)
