"""Native CPU rasteriser (shared math with the sm_100a kernels) against the PyTorch oracle."""
import pytest
import torch

from helpers import activated, assert_mostly_close, native_render, oracle_render, small_scene
from retinags_b200.data import synthetic
from retinags_b200.ops import oracle, rasterize


@pytest.mark.parametrize("deg", [0, 1, 3])
def test_forward_matches_oracle(deg):
    g, cams = small_scene(sh_degree=deg)
    for cam in cams[:2]:
        out, task, _, _ = native_render(g, cam, deg, want_depth=True)
        C, T, D, info = oracle_render(g, cam, deg)
        assert task.n_vis > 50
        torch.testing.assert_close(out[..., :3].permute(2, 0, 1), C, atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(out[..., 3], T, atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(task.depth, D, atol=1e-4, rtol=1e-4)


def test_binning_variants_agree():
    g, cams = small_scene(n=1500)
    a, ta, _, _ = native_render(g, cams[2], 3, binning="depth_first")
    b, tb, _, _ = native_render(g, cams[2], 3, binning="keyed")
    # the depth-first pipeline also drops tiles without a contributing pixel: fewer instances, same image
    assert torch.equal(a, b) and ta.n_inst <= tb.n_inst and ta.n_vis == tb.n_vis


def test_tight_rect_is_exact():
    g, cams = small_scene(n=1500)
    a, ta, _, _ = native_render(g, cams[0], 3, tight=True)
    b, tb, _, _ = native_render(g, cams[0], 3, tight=False)
    c, tc, _, _ = native_render(g, cams[0], 3, tight=2)  # per-tile test on top
    assert torch.equal(a, b) and torch.equal(a, c)
    assert tc.n_inst < ta.n_inst < tb.n_inst


def test_box_split_composites_to_whole():
    g, cams = small_scene(n=1500)
    big = 1e9
    whole, _, _, _ = native_render(g, cams[1], 3)
    left, _, _, _ = native_render(g, cams[1], 3, box=([-big, -big, -big], [0.1, big, big]))
    right, _, _, _ = native_render(g, cams[1], 3, box=([0.1, -big, -big], [big, big, big]))
    # which half is in front depends on the camera; composite both orders and take the matching one
    def over(f, b):
        return f[..., :3] + f[..., 3:4] * b[..., :3], f[..., 3] * b[..., 3]
    center = cams[1].camera_center
    first, second = (left, right) if center[0] <= 0.1 else (right, left)
    C, T = over(first, second)
    # the sort order inside one pixel differs only by which sub-model a splat belongs to, so the
    # composite equals the whole render up to float rounding, except where the T<1e-4 stop differs
    # (a pixel that stops in the whole render may keep blending across the two halves: |dT| < 1e-3)
    torch.testing.assert_close(C, whole[..., :3], atol=1e-3, rtol=0)
    torch.testing.assert_close(T, whole[..., 3], atol=1e-3, rtol=0)
    assert ((T - whole[..., 3]).abs() > 1e-5).float().mean() < 0.02


def test_backward_matches_autograd():
    deg = 3
    g, cams = small_scene(n=400, seed=5)
    cam = cams[0]
    box = ([-0.3, -1e9, -1e9], [1e9, 1e9, 1e9])
    a = activated(g)
    leaves = {k: v.clone().requires_grad_(True) for k, v in a.items()}
    C, T, D, _ = oracle.rasterize(cam, leaves["xyz"], leaves["sh"].view(-1, 16, 3), leaves["opacity"], leaves["scale"],
                                  leaves["rot"], deg, box[0], box[1])
    gen = torch.Generator().manual_seed(0)
    wC = torch.randn(C.shape, generator=gen)
    wT = torch.randn(T.shape, generator=gen)
    ((C * wC).sum() + (T * wT).sum()).backward()

    out, task, seg, c = native_render(a, cam, deg, box=box, raw=False)
    n = seg.count
    for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1), ("g_mean2d", 2)):
        setattr(seg, name, torch.zeros(n, w))
    grad = torch.cat([wC.permute(1, 2, 0), wT[..., None]], dim=-1).contiguous()
    task.backward(grad, [seg])
    for name, key in (("g_xyz", "xyz"), ("g_sh", "sh"), ("g_scale", "scale"), ("g_rot", "rot"), ("g_opacity", "opacity")):
        ref = leaves[key].grad
        got = getattr(seg, name)
        scale = ref.abs().max().item() + 1e-12
        err = (got - ref).abs().max().item() / scale
        assert err < 2e-3, (name, err, scale)


def test_raw_param_gradients():
    """Gradients with respect to raw parameters == autograd through the activations."""
    deg = 2
    g, cams = small_scene(n=300, seed=9, sh_degree=deg)
    cam = cams[2]
    leaves = {k: v.clone().requires_grad_(True) for k, v in g.items()}
    act = activated(leaves)
    C, T, D, _ = oracle.rasterize(cam, act["xyz"], act["sh"].view(-1, 16, 3), act["opacity"], act["scale"], act["rot"], deg)
    gen = torch.Generator().manual_seed(1)
    wC = torch.randn(C.shape, generator=gen)
    ((C * wC).sum()).backward()
    out, task, seg, c = native_render(g, cam, deg, raw=True)
    n = seg.count
    for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1)):
        setattr(seg, name, torch.zeros(n, w))
    seg.stat_grad = torch.zeros(n)
    seg.stat_denom = torch.zeros(n)
    seg.stat_maxrad = torch.zeros(n)
    grad = torch.cat([wC.permute(1, 2, 0), torch.zeros(C.shape[1], C.shape[2], 1)], dim=-1).contiguous()
    task.backward(grad, [seg])
    for name, key in (("g_xyz", "xyz"), ("g_sh", "sh"), ("g_scale", "scale"), ("g_rot", "rot"), ("g_opacity", "opacity")):
        ref = leaves[key].grad
        got = getattr(seg, name)
        scale = ref.abs().max().item() + 1e-12
        assert (got - ref).abs().max().item() / scale < 2e-3, name
    assert int(seg.stat_denom.sum()) == task.n_vis
    assert seg.stat_maxrad.max() > 0


def test_autograd_function_interface():
    g, cams = small_scene(n=300, seed=11)
    cam = cams[0]
    a = activated(g)
    st = rasterize.GaussianRasterizationSettings(
        image_height=cam.height, image_width=cam.width, tanfovx=cam.tan_fovx, tanfovy=cam.tan_fovy,
        bg=torch.tensor([0.2, 0.3, 0.4]), scale_modifier=1.0, viewmatrix=torch.tensor(cam.world_view_transform),
        projmatrix=torch.tensor(cam.full_proj_transform), projmatrix_inv=torch.tensor(cam.view_world_transform),
        range_low=torch.tensor([-1e9] * 3), range_up=torch.tensor([1e9] * 3), sh_degree=3,
        campos=torch.tensor(cam.camera_center))
    xyz = a["xyz"].clone().requires_grad_(True)
    m2d = torch.zeros(xyz.shape[0], 3, requires_grad=True)
    color, depth, alpha, radii = rasterize.GaussianRasterizer(st)(
        xyz, m2d, a["opacity"], shs=a["sh"].view(-1, 16, 3), scales=a["scale"], rotations=a["rot"])
    C, T, D, info = oracle_render(g, cam, 3)
    torch.testing.assert_close(color, C + T[None] * st.bg.view(3, 1, 1), atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(alpha[0], 1 - T, atol=2e-5, rtol=1e-4)
    assert torch.equal(radii > 0, info["radii"] > 0)
    color.sum().backward()
    assert xyz.grad.abs().sum() > 0 and m2d.grad.abs().sum() > 0
    vis = rasterize.GaussianRasterizer(st).markVisible(a["xyz"])
    view = torch.cat([a["xyz"], torch.ones(a["xyz"].shape[0], 1)], 1) @ torch.tensor(cam.world_view_transform)
    assert torch.equal(vis, view[:, 2] > 0.2)


def _slab_render(g, cam, slabs, frac=32, inst_per_gaussian=4.0, min_inst=1 << 16, check=True):
    import torch
    from retinags_b200.ops import rasterize
    seg = rasterize.Segment(*(g[k].contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
    task = rasterize.RenderTask("cpu", inst_per_gaussian=inst_per_gaussian, min_inst=min_inst)
    task.slabs, task.slab_frac256 = slabs, frac
    c = rasterize.make_camera(cam, 3)
    if check:
        out = task.forward(c, [seg], want_depth=True, check=True).clone()
    else:  # the training pattern: unchecked forwards, capacities adapted by poll() between steps
        for _ in range(6):
            out = task.forward(c, [seg], want_depth=True).clone()
            if not task.poll()["overflow"]:
                break
        else:
            raise AssertionError("capacities did not settle")
        task.n_inst = task.poll()["n_inst"]
    n = seg.count
    for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1)):
        setattr(seg, name, torch.zeros(n, w))
    grad = torch.randn(cam.height, cam.width, 4, generator=torch.Generator().manual_seed(2))
    task.backward(grad, [seg])
    grads = torch.cat([seg.g_xyz, seg.g_sh, seg.g_scale, seg.g_rot, seg.g_opacity], dim=1)
    return out, task.n_contrib.clone(), task.depth.clone(), task.n_inst, grads


def test_two_slab_forward_equals_single_pass_on_cpu():
    """Near slab first, far slab only for unsaturated tiles (CPU twins of the slab entry points): identical image, depth,
    contributor indices and gradients, fewer instances; also with buffers that start far too small, with unchecked
    forwards whose capacities poll() adapts, and with extreme slab fractions."""
    import torch
    from retinags_b200.data import synthetic
    g = synthetic.uniform_gaussians(30000, 5, sh_degree=3, log_scale_mean=-2.6)
    g["opacity"] = g["opacity"] + 4.0
    cam = synthetic.ring_cameras(3, 3.0, 160, 112)[1]
    ref = _slab_render(g, cam, False)
    assert (ref[0][..., 3] < 1e-3).float().mean() > 0.3  # the scene saturates
    cases = [dict(frac=32), dict(frac=12), dict(frac=200), dict(frac=0), dict(frac=256),
             dict(frac=32, inst_per_gaussian=0.01, min_inst=1024), dict(frac=12, inst_per_gaussian=0.01, min_inst=1024),
             dict(frac=32, inst_per_gaussian=0.01, min_inst=1024, check=False)]
    for kw in cases:
        got = _slab_render(g, cam, True, **kw)
        assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2]), kw
        assert torch.equal(got[4], ref[4]), kw
        assert got[3] <= ref[3], kw
    assert _slab_render(g, cam, True, frac=64)[3] < 0.8 * ref[3]


def test_two_slab_capacities_follow_changing_views():
    """One task, several cameras in turn, unchecked forwards: whenever poll() reports an overflow the render is repeated
    (as the trainer's warm-up does); every settled render equals the single-pass render."""
    import torch
    from retinags_b200.data import synthetic
    from retinags_b200.ops import rasterize
    g = synthetic.uniform_gaussians(30000, 7, sh_degree=3, log_scale_mean=-2.6)
    g["opacity"] = g["opacity"] + 4.0
    cams = synthetic.ring_cameras(4, 3.0, 160, 112) + synthetic.ring_cameras(2, 1.2, 160, 112)
    seg = rasterize.Segment(*(g[k].contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
    slab = rasterize.RenderTask("cpu", inst_per_gaussian=0.01, min_inst=1024)
    slab.slabs, slab.slab_frac256 = True, 48
    single = rasterize.RenderTask("cpu")
    renders = 0
    for cam in cams:
        c = rasterize.make_camera(cam, 3)
        ref = single.forward(c, [seg], check=True).clone()
        for _ in range(5):
            out = slab.forward(c, [seg]).clone()
            renders += 1
            if not slab.poll()["overflow"]:
                break
        else:
            raise AssertionError("capacities did not settle")
        assert torch.equal(out, ref)
        assert torch.equal(slab.n_contrib, single.n_contrib)
    assert renders <= len(cams) + 6


def test_training_steps_are_identical_with_two_slabs(monkeypatch):
    """Whole training steps (two local sub-models, compositing, loss, backward, Adam) with and without the two-slab
    forward: identical loss sums and parameters."""
    import torch
    from retinags_b200.bench_session import BenchSession

    def run(slabs):
        monkeypatch.setenv("RGS_SLABS", "1" if slabs else "0")
        monkeypatch.setenv("RGS_SLAB_FRACTION", "64")
        monkeypatch.setenv("RGS_OCCLUSION", "0")  # culling between the two sub-models is not bit-neutral: tested elsewhere
        sess = BenchSession("cpu", 0, 1, 30000, 160, 112, batch=2, n_views=4, gt_gaussians=3000, seed=3, sh_degree=2,
                            grid=(32, 32, 1), bvh_depth=1, scene_kind="uniform")
        for st in sess.stores.values():
            st.views()["opacity"].add_(3.0)  # opaque enough for tiles to saturate
        sums = []
        for it in range(3):
            res = sess.engine.train_step(*sess._batch(it), sess.sh_degree, sess.lrs)
            sess.settle()
            sums.append(torch.stack(res.sums).clone())
        active = any(t._slab_active for t in sess.engine._tasks.values())
        return sums, torch.cat([st.records() for st in sess.stores.values()]), active

    a, pa, used_a = run(False)
    b, pb, used_b = run(True)
    assert used_b and not used_a
    for x, y in zip(a, b):
        torch.testing.assert_close(x, y, rtol=1e-11, atol=1e-8)  # the loss sums are OpenMP reductions
    assert torch.equal(pa, pb)


def test_gradients_against_finite_differences():
    """Central differences of a scalar function of the native render, for the parameters with the largest analytic
    gradient of every group (raw parameters, so the activation chain rules are included)."""
    deg = 2
    g, cams = small_scene(n=120, seed=9, width=48, height=32)
    cam = cams[0]
    gen = torch.Generator().manual_seed(4)
    weight = torch.randn(cam.height, cam.width, 4, generator=gen)

    def value(params):
        out, _, _, _ = native_render(params, cam, deg)
        return float((out.double() * weight.double()).sum())

    out, task, seg, c = native_render(g, cam, deg)
    n = seg.count
    for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1)):
        setattr(seg, name, torch.zeros(n, w))
    task.backward(weight.contiguous(), [seg])
    checked = 0
    for name, key, steps in (("g_xyz", "xyz", (2e-4, 1e-3, 5e-3)), ("g_scale", "scale", (1e-3, 5e-3, 2e-2)),
                             ("g_rot", "rot", (1e-3, 5e-3, 2e-2)), ("g_opacity", "opacity", (2e-3, 1e-2, 5e-2)),
                             ("g_sh", "sh", (2e-3, 1e-2, 5e-2))):
        analytic = getattr(seg, name)
        flat = analytic.abs().flatten()
        for idx in flat.topk(3).indices.tolist():
            i, j = divmod(idx, analytic.shape[1])
            an = float(analytic[i, j])
            errs = []
            for eps in steps:
                plus = {k: v.clone() for k, v in g.items()}
                minus = {k: v.clone() for k, v in g.items()}
                plus[key][i, j] += eps
                minus[key][i, j] -= eps
                fd = (value(plus) - value(minus)) / (2 * eps)
                errs.append(abs(fd - an) / max(abs(an), abs(fd), 1e-9))
            # The render has jumps (alpha threshold 1/255, integer radius, stop rule): a jump inside [-eps, eps] spoils that
            # difference quotient by jump / (2 eps), so one of three step sizes has to agree, not all of them.
            assert min(errs) < 0.06, (name, i, j, an, errs)
            checked += 1
    assert checked == 15


def test_depth_gradient_matches_autograd():
    """A loss on the depth output reaches means, scales, rotations and opacities like autograd through the oracle's
    D = sum z_i alpha_i T_i (the reference's dL/ddepth path), alone and together with a colour loss."""
    deg = 1
    g, cams = small_scene(n=300, seed=13, sh_degree=deg)
    cam = cams[1]
    a = activated(g)
    gen = torch.Generator().manual_seed(2)
    for with_colour in (False, True):
        leaves = {k: v.clone().requires_grad_(True) for k, v in a.items()}
        C, T, D, _ = oracle.rasterize(cam, leaves["xyz"], leaves["sh"].view(-1, 16, 3), leaves["opacity"], leaves["scale"],
                                      leaves["rot"], deg)
        wD = torch.randn(D.shape, generator=gen)
        wC = torch.randn(C.shape, generator=gen) if with_colour else torch.zeros(C.shape)
        ((D * wD).sum() + (C * wC).sum()).backward()
        out, task, seg, c = native_render(a, cam, deg, raw=False, want_depth=True)
        torch.testing.assert_close(task.depth, D.detach(), atol=2e-5, rtol=1e-4)
        n = seg.count
        for name, w in (("g_xyz", 3), ("g_sh", 48), ("g_scale", 3), ("g_rot", 4), ("g_opacity", 1)):
            setattr(seg, name, torch.zeros(n, w))
        grad = torch.cat([wC.permute(1, 2, 0), torch.zeros(C.shape[1], C.shape[2], 1)], dim=-1).contiguous()
        task.backward(grad, [seg], grad_depth=wD.contiguous())
        for name, key in (("g_xyz", "xyz"), ("g_scale", "scale"), ("g_rot", "rot"), ("g_opacity", "opacity")):
            ref = leaves[key].grad
            got = getattr(seg, name)
            scale = ref.abs().max().item() + 1e-12
            assert (got - ref).abs().max().item() / scale < 2e-3, (name, with_colour)
    # the autograd interface no longer drops the depth gradient
    st = rasterize.GaussianRasterizationSettings(
        image_height=cam.height, image_width=cam.width, tanfovx=cam.tan_fovx, tanfovy=cam.tan_fovy,
        bg=torch.zeros(3), scale_modifier=1.0, viewmatrix=torch.tensor(cam.world_view_transform),
        projmatrix=torch.tensor(cam.full_proj_transform), projmatrix_inv=torch.tensor(cam.view_world_transform),
        range_low=torch.tensor([-1e9] * 3), range_up=torch.tensor([1e9] * 3), sh_degree=deg,
        campos=torch.tensor(cam.camera_center))
    xyz = a["xyz"].clone().requires_grad_(True)
    _, depth, _, _ = rasterize.GaussianRasterizer(st)(xyz, torch.zeros(xyz.shape[0], 3), a["opacity"],
                                                      shs=a["sh"].view(-1, 16, 3)[:, :4], scales=a["scale"], rotations=a["rot"])
    (depth[0] * wD).sum().backward()
    ref = leaves["xyz"].grad if not with_colour else None
    leaves = {k: v.clone().requires_grad_(True) for k, v in a.items()}
    _, _, D, _ = oracle.rasterize(cam, leaves["xyz"], leaves["sh"].view(-1, 16, 3), leaves["opacity"], leaves["scale"],
                                  leaves["rot"], deg)
    (D * wD).sum().backward()
    ref = leaves["xyz"].grad
    assert (xyz.grad - ref).abs().max().item() / (ref.abs().max().item() + 1e-12) < 2e-3


def test_tiny_instance_capacity_regrows_with_two_slabs():
    """An instance buffer far smaller than one slab needs (256 entries): both slab regions stay inside it, the render
    reports the overflow, grows and ends with the image of a comfortably sized task."""
    g = synthetic.uniform_gaussians(20000, 4, sh_degree=3, log_scale_mean=-3.6)
    cam = synthetic.ring_cameras(3, 3.0, 320, 208)[0]
    ref, _, _, _ = native_render(g, cam, 3)
    for frac in (6, 32, 200):
        seg = rasterize.Segment(*(g[k].contiguous() for k in ("xyz", "sh", "scale", "rot", "opacity")))
        task = rasterize.RenderTask("cpu", inst_per_gaussian=0.01, min_inst=256)
        task.slabs, task.slab_frac256 = True, frac
        out = task.forward(rasterize.make_camera(cam, 3), [seg], check=True)
        assert task._slab_active and task.cap_inst > 256
        cap_a, cap_b = task._slab_regions()
        assert 0 < cap_a < task.cap_inst and cap_a + cap_b == task.cap_inst
        assert_mostly_close(out, ref, atol=1e-5, rtol=1e-4)
