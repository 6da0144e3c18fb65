"""Compositing + L1/D-SSIM forward and hand-written backward against autograd (CPU)."""
import torch

from retinags_b200.ops import oracle
from retinags_b200.ops.loss import CompositeLoss


def _partials(K, H, W, seed=0):
    g = torch.Generator().manual_seed(seed)
    parts = []
    for _ in range(K):
        T = torch.rand(H, W, 1, generator=g) * 0.9 + 0.05
        C = torch.rand(H, W, 3, generator=g) * (1 - T)
        parts.append(torch.cat([C, T], dim=-1).contiguous())
    return parts


def test_composite_loss_matches_autograd():
    H, W, K = 45, 70, 3
    parts = _partials(K, H, W)
    gt = torch.rand(3, H, W, generator=torch.Generator().manual_seed(5))
    bg = (0.1, 0.2, 0.3)
    leaves = [p.clone().requires_grad_(True) for p in parts]
    img, T = oracle.composite([p[..., :3].permute(2, 0, 1) for p in leaves], [p[..., 3] for p in leaves], bg)
    loss = oracle.training_loss(img, gt, 0.2)
    loss.backward()

    cl = CompositeLoss("cpu", H, W)
    image, trans = cl.composite(parts, bg)
    torch.testing.assert_close(image, img.detach(), atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(trans, T.detach(), atol=1e-6, rtol=1e-5)
    sums = cl.loss(gt, 0.2)
    got = cl.loss_from_sums(sums, 0.2)
    assert abs(got["loss"] - loss.item()) < 1e-5
    grads = [torch.zeros_like(p) for p in parts]
    cl.backward(parts, grads, bg)
    for k in range(K):
        ref = leaves[k].grad
        assert (grads[k] - ref).abs().max().item() < 2e-3 * ref.abs().max().item() + 1e-9


def test_row_bands_equal_whole_image():
    H, W, K = 64, 48, 2
    parts = _partials(K, H, W, seed=2)
    gt = torch.rand(3, H, W, generator=torch.Generator().manual_seed(6))
    bg = (0.0, 0.0, 0.0)
    whole = CompositeLoss("cpu", H, W)
    whole.composite(parts, bg)
    s_whole = whole.loss(gt).clone()
    g_whole = [torch.zeros_like(p) for p in parts]
    whole.backward(parts, g_whole, bg)

    g_band = [torch.zeros_like(p) for p in parts]
    s_total = torch.zeros(3, dtype=torch.float64)
    for r0, r1 in ((0, 16), (16, 48), (48, 64)):
        band = CompositeLoss("cpu", H, W)
        band.composite(parts, bg, max(0, r0 - 10), min(H, r1 + 10))
        s_total += band.loss(gt, row0=r0, row1=r1)
        band.backward(parts, g_band, bg, r0, r1)
    torch.testing.assert_close(s_total, s_whole, atol=1e-4, rtol=1e-6)
    for a, b in zip(g_band, g_whole):
        torch.testing.assert_close(a, b, atol=1e-9, rtol=1e-5)


def test_fused_training_path_equals_separate_steps():
    """composite + loss + backward in two calls == the four separate steps, on a row band of three partials."""
    import torch
    from retinags_b200.ops.loss import CompositeLoss
    g = torch.Generator().manual_seed(5)
    H, W, K = 70, 90, 3
    parts = [torch.cat([torch.rand(H, W, 3, generator=g) * 0.4, torch.rand(H, W, 1, generator=g)], dim=2).contiguous()
             for _ in range(K)]
    gt = torch.rand(3, H, W, generator=g)
    bg = (0.1, 0.2, 0.3)
    for rows in ((0, H), (16, 48)):
        a, b = CompositeLoss("cpu", H, W), CompositeLoss("cpu", H, W)
        ga = [torch.zeros(H, W, 4) for _ in range(K)]
        gb = [torch.zeros(H, W, 4) for _ in range(K)]
        a.composite(parts, bg, max(0, rows[0] - 10), min(H, rows[1] + 10))
        sa = a.loss(gt, 0.2, rows[0], rows[1]).clone()
        a.backward(parts, ga, bg, rows[0], rows[1])
        sb = b.fused_loss_backward(parts, gb, gt, bg, 0.2, rows[0], rows[1]).clone()
        torch.testing.assert_close(sa, sb, rtol=1e-10, atol=1e-9)  # the sums are OpenMP reductions
        for x, y in zip(ga, gb):
            assert torch.equal(x, y)
        assert float(sum(x.abs().sum() for x in gb)) > 0


def test_partials_behind_saturated_ones_get_exactly_zero_gradient():
    """Where the partials in front leave less than 1e-4 of transmittance, the partials behind receive zero instead of
    a gradient scaled by that factor (both backward paths); everywhere else the gradients are those of autograd."""
    H, W, K = 40, 48, 3
    parts = _partials(K, H, W, seed=3)
    parts[0][:20, :, 3] = 5e-5      # the front partial saturates the upper half
    parts[1][30:, 10:20, 3] = 0.0   # the second one a patch of the lower half (exactly opaque)
    gt = torch.rand(3, H, W, generator=torch.Generator().manual_seed(7))
    bg = (0.2, 0.1, 0.3)
    leaves = [p.clone().requires_grad_(True) for p in parts]
    img, _ = oracle.composite([p[..., :3].permute(2, 0, 1) for p in leaves], [p[..., 3] for p in leaves], bg)
    oracle.training_loss(img, gt, 0.2).backward()
    for fused in (False, True):
        cl = CompositeLoss("cpu", H, W)
        grads = [torch.full_like(p, 7.0) for p in parts]
        if fused:
            cl.fused_loss_backward(parts, grads, gt, bg, 0.2)
        else:
            cl.composite(parts, bg)
            cl.loss(gt, 0.2)
            cl.backward(parts, grads, bg)
        assert float(grads[1][:20].abs().max()) == 0.0 and float(grads[2][:20].abs().max()) == 0.0
        assert float(grads[2][30:, 10:20].abs().max()) == 0.0
        assert float(grads[0].abs().max()) > 0 and float(grads[1][20:].abs().max()) > 0
        keep = torch.ones(H, W, dtype=torch.bool)
        keep[:20] = False
        for k in range(K):
            ref = leaves[k].grad
            m = keep.clone() if k > 0 else torch.ones(H, W, dtype=torch.bool)
            if k == 2:
                m[30:, 10:20] = False
            assert (grads[k] - ref)[m].abs().max().item() < 2e-3 * ref.abs().max().item() + 1e-9


def test_finished_mark_in_the_transmittance_blocks_the_partials_behind():
    """``CompositeLoss.marked``: the lowest mantissa bit of a partial's transmittance says "this pixel is finished"
    (``rgs_mark_finished`` in the blend kernels); the partials behind it get zero. Unmarked use ignores the bit."""
    H, W, K = 24, 32, 3
    parts = _partials(K, H, W, seed=4)
    for p in parts:  # clear the low bits of random data, then mark the upper half of the middle partial as finished
        bits = p[..., 3].contiguous().view(torch.int32) & ~1
        p[..., 3] = bits.view(torch.float32)
    bits = parts[1][..., 3].contiguous().view(torch.int32)
    bits[:12] |= 1
    parts[1][..., 3] = bits.view(torch.float32)
    gt = torch.rand(3, H, W, generator=torch.Generator().manual_seed(8))
    bg = (0.3, 0.3, 0.1)
    out = {}
    for marked in (False, True):
        cl = CompositeLoss("cpu", H, W)
        cl.marked = marked
        grads = [torch.zeros_like(p) for p in parts]
        cl.fused_loss_backward(parts, grads, gt, bg, 0.2)
        out[marked] = grads
    assert float(out[True][2][:12].abs().max()) == 0.0 and float(out[False][2][:12].abs().max()) > 0.0
    for k in range(K):
        rows = slice(12, None) if k == 2 else slice(None)
        assert torch.equal(out[True][k][rows], out[False][k][rows])
