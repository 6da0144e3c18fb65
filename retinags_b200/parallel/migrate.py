"""Migration of Gaussians between sub-models after the partition changed.

Each Gaussian moves, with its Adam moments, to the sub-model whose new box contains its centre: a
177-float record ``[params(59), exp_avg(59), exp_avg_sq(59)]`` per Gaussian
(``scene/gaussian_nn_module.py:832-936``, ``basic_parallel_trainer/result_aggregator.py:150-190``,
``trainer4tree_partition.py:290-317``).  Records are produced one source sub-model at a time and in
bounded chunks, so the peak extra memory is one chunk per peer rather than a full copy of the model
(the reference warns about running out of memory here, ``trainer4tree_partition.py:681-682``).
The per-pair counts travel as one all-reduce of an (M,M) matrix; records that stay on the rank are
appended directly.  Records that change rank travel in one of two ways:

* ``path="peer"`` (CUDA ranks of one node): the pack kernel (``csrc/rgs_surgery.cu``) gathers the rows from the
  source's column groups and stores the 177-float records straight into the destination rank's inbox, a
  peer-mapped region (``parallel/peer.py``); one source sub-model per round, so the inbox holds at most one
  sub-model; the destination unpacks from its own memory after the round's barrier.  No NCCL call moves
  Gaussian bytes.
* ``path="dist"``: ``torch.distributed`` send/recv of packed chunks (gloo ranks, several nodes).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import native

from ..models.gaussians import RECORD, GaussianStore

CHUNK_ROWS = 1 << 20


def migrate(old: dict[int, GaussianStore], tree, lo, hi, model2rank, rank: int, world: int, device, sh_degree: int,
            group=None, path: str = "auto") -> dict[int, GaussianStore]:
    M = len(model2rank)
    device = torch.device(device)
    if path == "auto":
        path = "peer" if (device.type == "cuda" and world > 1 and os.environ.get("RGS_MIGRATE_PATH", "peer") == "peer") else "dist"
    local_new = [m for m in range(M) if model2rank[m] == rank]
    # destination of every resident Gaussian
    dest = {s: tree.label(st.xyz) if st.count else torch.zeros(0, dtype=torch.int64, device=device) for s, st in old.items()}
    counts = torch.zeros(M, M, dtype=torch.int64, device=device)
    for s, d in dest.items():
        if d.numel():
            counts[s] = torch.bincount(d, minlength=M)
    if world > 1:
        dist.all_reduce(counts, group=group)
    counts = counts.cpu()
    step = max(st.step for st in old.values()) if old else 0
    new = {m: GaussianStore(max(int(counts[:, m].sum()), 4), device, sh_degree, lo[m], hi[m], m) for m in local_new}
    for st in new.values():
        st.step = step
    old_rank_of = {s: r for s, r in enumerate(model2rank)}  # sub-model ids keep their rank (i % world)
    if path == "peer" and world > 1:
        _move_peer(old, new, dest, counts, model2rank, rank, world, device, group)
        return new
    for s in range(M):
        for d in range(M):
            n = int(counts[s, d])
            if n == 0:
                continue
            rs, rd = old_rank_of[s], model2rank[d]
            if rs != rank and rd != rank:
                continue
            idx = (dest[s] == d).nonzero(as_tuple=True)[0] if rs == rank else None
            for c0 in range(0, n, CHUNK_ROWS):
                c1 = min(n, c0 + CHUNK_ROWS)
                if rs == rank:
                    rec = old[s].migration_records(idx[c0:c1]).contiguous()
                    if rd == rank:
                        new[d].append_migration(rec)
                    else:
                        dist.send(rec, rd, group=group)
                else:
                    buf = torch.empty(c1 - c0, 3 * RECORD, dtype=torch.float32, device=device)
                    dist.recv(buf, rs, group=group)
                    new[d].append_migration(buf)
        if s in old:
            old[s].count = 0  # release the source as soon as it has been drained
    return new


def _move_peer(old, new, dest, counts, model2rank, rank, world, device, group):
    """One round per source sub-model: its owner packs the rows of every destination straight into the destination
    rank's inbox (peer stores), everybody synchronises, destinations unpack from their own memory."""
    from .peer import PeerRegion
    M = len(model2rank)
    row_bytes = 3 * RECORD * 4

    def inbox_rows(s, r):  # rows that round s delivers to rank r from another rank
        return sum(int(counts[s, d]) for d in range(M) if model2rank[d] == r and model2rank[s] != r)

    need = max([inbox_rows(s, r) for s in range(M) for r in range(world)] + [1])
    region = PeerRegion(need * row_bytes, device, group)
    try:
        for s in range(M):
            rs = model2rank[s]
            offset = {}
            for r in range(world):
                run = 0
                for d in range(M):
                    if model2rank[d] == r and rs != r:
                        offset[d] = run
                        run += int(counts[s, d])
            if rs == rank and s in old:
                st = old[s]
                for d in range(M):
                    n = int(counts[s, d])
                    if n == 0:
                        continue
                    idx = (dest[s] == d).nonzero(as_tuple=True)[0].contiguous()
                    rd = model2rank[d]
                    if rd == rank:
                        for c0 in range(0, n, CHUNK_ROWS):
                            new[d].append_migration(st.migration_records(idx[c0:c0 + CHUNK_ROWS]))
                    else:
                        out = region.ptrs[rd] + offset[d] * row_bytes
                        native.call("records_pack", device, st.params, st.exp_avg, st.exp_avg_sq, st.cap, idx, 0, n, out)
            torch.cuda.synchronize(device)
            dist.barrier(group)  # the round's records have landed
            if rs != rank:
                for d in range(M):
                    n = int(counts[s, d])
                    if n and model2rank[d] == rank:
                        new[d].append_migration(region.view(offset[d] * row_bytes, (n, 3 * RECORD)))
            if s in old:
                old[s].count = 0
            torch.cuda.synchronize(device)
            dist.barrier(group)  # inbox free for the next round
    finally:
        region.close()
