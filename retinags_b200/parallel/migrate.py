"""Migration of Gaussians between sub-models after the partition changed.

Each Gaussian moves, with its Adam moments, to the sub-model whose new box contains its centre: a
177-float record ``[params(59), exp_avg(59), exp_avg_sq(59)]`` per Gaussian
(``scene/gaussian_nn_module.py:832-936``, ``basic_parallel_trainer/result_aggregator.py:150-190``,
``trainer4tree_partition.py:290-317``).  Records are produced one source sub-model at a time and in
bounded chunks, so the peak extra memory is one chunk per peer rather than a full copy of the model
(the reference warns about running out of memory here, ``trainer4tree_partition.py:681-682``).
The per-pair counts travel as one all-reduce of an (M,M) matrix, the records as point-to-point
messages; records that stay on the rank are appended directly.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.gaussians import RECORD, GaussianStore

CHUNK_ROWS = 1 << 20


def migrate(old: dict[int, GaussianStore], tree, lo, hi, model2rank, rank: int, world: int, device, sh_degree: int,
            group=None) -> dict[int, GaussianStore]:
    M = len(model2rank)
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
