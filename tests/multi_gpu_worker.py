"""Worker of tests/test_multi_gpu.py (launched by torch.distributed.run, one rank per GPU)."""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _check_migration(sess, rank, world, dev) -> bool:
    """Repartition with the other split order: the peer-store path and the send/recv path build identical sub-models,
    and no Gaussian is lost."""
    from retinags_b200.models.gaussians import GaussianStore
    from retinags_b200.parallel.migrate import migrate
    from retinags_b200.parallel.partition import BvhTree

    tree2 = BvhTree.build(sess.tree.grid, sess.bvh_depth, (1, 0))
    lo, hi = tree2.leaf_boxes_world(open_border=True)

    def clones():
        out = {}
        for m, st in sess.stores.items():
            c = GaussianStore(max(st.count, 4), dev, st.max_sh_degree, st.box_lo, st.box_hi, m)
            c.append_migration(st.migration_records())
            c.step = st.step
            out[m] = c
        return out

    before = torch.tensor([sum(st.count for st in sess.stores.values())], device=dev)
    a = migrate(clones(), tree2, lo, hi, sess.model2rank, rank, world, dev, 3, None, path="peer")
    b = migrate(clones(), tree2, lo, hi, sess.model2rank, rank, world, dev, 3, None, path="dist")
    after = torch.tensor([sum(st.count for st in a.values())], device=dev)
    moved = torch.tensor([sum(int((tree2.label(st.xyz) != m).sum()) for m, st in sess.stores.items())], device=dev)
    for t in (before, after, moved):
        dist.all_reduce(t)
    same = all(a[m].count == b[m].count and torch.equal(a[m].migration_records(), b[m].migration_records()) for m in a)
    inside = all(bool((tree2.label(st.xyz) == m).all()) for m, st in a.items() if st.count)
    good = torch.tensor([int(same and inside)], device=dev)
    dist.all_reduce(good, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"migration: {int(moved)} of {int(before)} Gaussians change sub-model; paths identical on every rank: "
              f"{bool(good.item())}", flush=True)
    return bool(good.item()) and int(before) == int(after) and int(moved) > 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--transport", default="peer")
    ap.add_argument("--out", default="")
    ap.add_argument("--occlusion", type=int, default=0)
    a = ap.parse_args()
    os.environ["RGS_OCCLUSION"] = str(a.occlusion)  # finished-tile maps exchanged between the ranks (training forward)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from retinags_b200.bench_session import BenchSession

    kw = dict(n_gaussians=300000, width=640, height=416, batch=2, n_views=6, gt_gaussians=60000, seed=2, sh_degree=3,
              grid=(128, 128, 1))
    sess = BenchSession(dev, rank, world, transport=a.transport, **kw)
    single = BenchSession(dev, 0, 1, bvh_depth=0, **kw) if rank == 0 else None
    ok = True
    for i in range(2):
        img, rows, _ = sess.render_view(i)
        full = torch.zeros_like(img)
        full[:, rows[0]:rows[1]] = img[:, rows[0]:rows[1]]
        dist.all_reduce(full)
        if rank == 0:
            ref, _, trans = single.render_view(i)
            diff = (full - ref).abs().max(0).values
            open_px = trans > 2e-3
            frac = (diff[open_px] > 2e-5).float().mean().item()
            print(f"view {i}: max diff {diff.max().item():.2e}, frac>2e-5 on open pixels {frac:.2e}", flush=True)
            ok &= frac < 5e-3 and diff.max().item() < 5e-3
    losses = []
    for it in range(4):
        loss, _, _ = sess.step_e2e(it % 3)
        t = torch.tensor([loss], dtype=torch.float64, device=dev)
        dist.all_reduce(t)
        losses.append(float(t))
    torch.cuda.synchronize()
    if hasattr(sess.engine.transport, "check"):
        sess.engine.transport.check()
    if rank == 0:
        ref_losses = [single.step_e2e(it % 3)[0] for it in range(4)]
        print("losses", losses, ref_losses, flush=True)
        ok &= all(abs(x - y) < 5e-4 * max(1.0, abs(y)) for x, y in zip(losses, ref_losses))
    ok &= _check_migration(sess, rank, world, dev)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    dist.barrier()
    if hasattr(sess.engine.transport, "close"):
        sess.engine.transport.close()
    if rank == 0 and bool(flag.item()):
        print("MULTI_GPU_OK", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if bool(flag.item()) else 1)


if __name__ == "__main__":
    main()
