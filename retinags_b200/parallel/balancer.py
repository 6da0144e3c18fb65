"""Greedy packing of the shuffled camera list into batches.

Parity: ``utils/workload_utils.py:6-59`` of the reference.  A camera costs one render task on the
rank of every sub-model it sees; a batch holds at most ``max_batch`` cameras and no rank gets more
than ``max_task`` render tasks (``--MAX_LOAD``), except that a batch is never empty.
"""
from __future__ import annotations

import numpy as np


class WorkloadBalancer:
    def __init__(self, num_rank: int, model2rank):
        self.num_rank = num_rank
        self.model2rank = list(model2rank)

    def load_per_rank(self, relation_row) -> np.ndarray:
        load = np.zeros(self.num_rank, dtype=np.int64)
        for m, r in enumerate(relation_row):
            if r >= 0:
                load[self.model2rank[m]] += 1
        return load

    def groups(self, relation: np.ndarray, order, max_task: int, max_batch: int) -> list[tuple]:
        out, cur, load = [], [], np.zeros(self.num_rank, dtype=np.int64)
        for idx in order:
            idx = int(idx)
            need = self.load_per_rank(relation[idx])
            if cur and (len(cur) >= max_batch or ((load + need) > max_task).any()):
                out.append(tuple(cur))
                cur, load = [], np.zeros(self.num_rank, dtype=np.int64)
            cur.append(idx)
            load = load + need
        if cur:
            out.append(tuple(cur))
        return out
