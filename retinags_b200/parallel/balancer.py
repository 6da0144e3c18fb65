"""Packing of the shuffled camera list into batches.

Parity: ``utils/workload_utils.py:6-59`` of the reference (``groups``).  A camera costs one render task on the
rank of every sub-model it sees; a batch holds at most ``max_batch`` cameras and no rank gets more
than ``max_task`` render tasks (``--MAX_LOAD``), except that a batch is never empty.

Beyond the reference: ``groups_balanced`` chooses *which* cameras share a batch.  A step lasts as long as its
busiest rank, and how busy a rank is depends on where the camera stands relative to the rank's sub-model, so
cameras whose loads complement each other are batched together.  The per-(camera, sub-model) cost comes from
``estimate_costs`` (a geometric estimate of the number of tile instances, from a strided sample of the Gaussians) or
from counters measured in an earlier epoch.  The set of cameras of an epoch and the batch limits are unchanged.
"""
from __future__ import annotations

import numpy as np
import torch


def estimate_costs(stores: dict, cams: list, num_models: int, stride: int = 64, tile: int = 16) -> np.ndarray:
    """(len(cams), num_models) estimated tile instances of every local sub-model in every camera (zeros for sub-models
    of other ranks: sum the matrices of all ranks).  Uses every ``stride``-th Gaussian: 3-sigma radius of the largest
    axis, pinhole projection, near plane 0.2, rectangle clipped to the image."""
    out = np.zeros((len(cams), num_models), dtype=np.float64)
    for m, st in stores.items():
        if st.count == 0:
            continue
        v = st.views()
        xyz = v["xyz"][::stride].double()
        smax = torch.exp(v["scale"][::stride]).max(dim=1).values.double()
        lo = torch.as_tensor(st.box_lo, dtype=torch.float64, device=xyz.device)
        hi = torch.as_tensor(st.box_hi, dtype=torch.float64, device=xyz.device)
        inside = ((xyz > lo) & (xyz <= hi)).all(dim=1)  # borrowed rows are not part of the store; guards stale rows
        for i, cam in enumerate(cams):
            w2c = torch.as_tensor(np.asarray(cam.world_view_transform).T.copy(), dtype=torch.float64, device=xyz.device)
            t = xyz @ w2c[:3, :3].T + w2c[:3, 3]
            z = t[:, 2]
            ok = inside & (z > 0.2)
            fx, fy = cam.width / (2.0 * cam.tan_fovx), cam.height / (2.0 * cam.tan_fovy)
            zc = z.clamp_min(0.2)
            px, py = t[:, 0] / zc * fx + 0.5 * cam.width, t[:, 1] / zc * fy + 0.5 * cam.height
            r = torch.ceil(3.0 * smax * max(fx, fy) / zc) + 1.0
            x0 = ((px - r) / tile).floor().clamp(0, -(-cam.width // tile))
            x1 = ((px + r) / tile).floor().add(1).clamp(0, -(-cam.width // tile))
            y0 = ((py - r) / tile).floor().clamp(0, -(-cam.height // tile))
            y1 = ((py + r) / tile).floor().add(1).clamp(0, -(-cam.height // tile))
            area = ((x1 - x0) * (y1 - y0)).clamp_min(0)
            out[i, m] = float((area * ok).sum()) * stride
    return out


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

    def groups_balanced(self, relation: np.ndarray, order, cost: np.ndarray, max_task: int, max_batch: int,
                        window: int = 64) -> list[tuple]:
        """Same limits as ``groups``, but every batch is completed with the camera (among the next ``window`` unused ones
        of ``order``) that keeps the busiest rank of the batch least busy.  ``cost``: (cameras, sub-models)."""
        order = [int(i) for i in order]
        rank_cost = np.zeros((relation.shape[0], self.num_rank), dtype=np.float64)
        for m, r in enumerate(self.model2rank):
            rank_cost[:, r] += np.where(relation[:, m] >= 0, cost[:, m], 0.0)
        used = [False] * len(order)
        out, first = [], 0
        while first < len(order):
            if used[first]:
                first += 1
                continue
            used[first] = True
            cur = [order[first]]
            tasks = self.load_per_rank(relation[cur[0]])
            load = rank_cost[cur[0]].copy()
            while len(cur) < max_batch:
                best, best_peak, seen = -1, None, 0
                for k in range(first + 1, len(order)):
                    if used[k]:
                        continue
                    seen += 1
                    if seen > window:
                        break
                    c = order[k]
                    if ((tasks + self.load_per_rank(relation[c])) > max_task).any():
                        continue
                    peak = float((load + rank_cost[c]).max())
                    if best_peak is None or peak < best_peak:
                        best, best_peak = k, peak
                if best < 0:
                    break
                used[best] = True
                c = order[best]
                cur.append(c)
                tasks = tasks + self.load_per_rank(relation[c])
                load = load + rank_cost[c]
            out.append(tuple(cur))
        return out

    def imbalance(self, relation: np.ndarray, groups, cost: np.ndarray) -> float:
        """Mean over batches of (busiest rank / average rank) under ``cost``: 1.0 is perfect balance."""
        vals = []
        for g in groups:
            load = np.zeros(self.num_rank)
            for c in g:
                for m, r in enumerate(self.model2rank):
                    if relation[c, m] >= 0:
                        load[r] += cost[c, m]
            if load.mean() > 0:
                vals.append(load.max() / load.mean())
        return float(np.mean(vals)) if vals else 1.0
