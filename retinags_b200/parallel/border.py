"""Border Gaussians: what a sub-model borrows from its neighbours.

A Gaussian whose extent ``mean +- 3 max(scale)`` reaches into another sub-model's box must also be
rasterised there (the half-Gaussian clip then keeps, per pixel, only the sub-model whose box holds the
ray sample).  Owners therefore lend such Gaussians to the sub-models they reach into and get the
gradients back before the optimiser step.

Parity: ``parallel_utils/basic_parallel_trainer/result_aggregator.py:55-147`` (candidate = extent
crosses the own box; per destination: extent overlaps its box), ``task_utils.py:230-362`` (62-float
activated rows forward, same shape backward) and ``trainer4tree_partition.py:354-388,521-571``.
Differences: rows carry the 59 *raw* parameters (the render kernel applies the activations itself, so
the returned gradients are already with respect to the raw parameters and are simply added to the
owner's gradient block); the selection can be cached for ``refresh_interval`` steps instead of being
recomputed by boolean masks every iteration; only the index lists are rebuilt, the rows are regathered
every step because parameters change.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..models.gaussians import NAMES, RECORD, WIDTHS, GaussianStore
from ..ops import native
from ..ops.rasterize import Segment

GRAD_COLS = RECORD + 1  # 59 parameter gradients + the screen-gradient statistic


def select_border(store: GaussianStore, m: int, lo: torch.Tensor, hi: torch.Tensor, margin: float = 0.0,
                  native_mask: bool | None = None) -> dict[int, torch.Tensor]:
    """Indices (ascending) of the Gaussians of sub-model ``m`` that are lent to every other sub-model d: the box
    centre +- 3 exp(max log-scale) (1 + margin) leaves the box of m and overlaps the box of d. ``lo``/``hi``: (M,3).

    ``native_mask``: one pass of the mask kernel (``csrc/rgs_border.cu``, ``rgs_border.h``) instead of boolean-mask
    gathers per destination; the default for up to 63 sub-models (``RGS_BORDER_SELECT=torch`` selects the masks)."""
    M = int(lo.shape[0])
    out: dict[int, torch.Tensor] = {}
    if store.count == 0 or M < 2:
        return out
    v = store.views()
    if native_mask is None:
        native_mask = os.environ.get("RGS_BORDER_SELECT", "native") == "native" and M <= 63
    if native_mask:
        boxes = torch.cat([lo, hi], dim=1).to(store.device, torch.float32).contiguous()
        masks = torch.empty(store.count, dtype=torch.int64, device=store.device)
        native.call("border_mask", store.device, v["xyz"], v["scale"], store.count, boxes, M, m, float(margin), masks,
                    sig="ppipiifpp")
        cand = masks.nonzero(as_tuple=True)[0]
        if cand.numel():
            # all destinations at once (three host round trips instead of two per destination): row d of `bits` marks
            # the candidates lent to d, and a boolean gather of the row-expanded candidates lists them destination by
            # destination, ascending inside each
            shifts = torch.arange(M, device=store.device, dtype=torch.int64).unsqueeze(1)
            bits = ((masks[cand].unsqueeze(0) >> shifts) & 1).bool()
            bits[m] = False
            counts = bits.sum(dim=1).tolist()
            flat = cand.unsqueeze(0).expand(M, -1)[bits]
            off = 0
            for d in range(M):
                if counts[d]:
                    out[d] = flat[off:off + counts[d]].contiguous()
                    off += counts[d]
        return out
    ext = 3.0 * torch.exp(v["scale"]).max(dim=1, keepdim=True).values * (1.0 + margin)
    blo, bhi = v["xyz"] - ext, v["xyz"] + ext
    cand = ((blo <= lo[m]) | (bhi > hi[m])).any(dim=1).nonzero(as_tuple=True)[0]
    if cand.numel() == 0:
        return out
    clo, chi = blo[cand], bhi[cand]
    for d in range(M):
        if d != m:
            idx = cand[((chi > lo[d]) & (clo <= hi[d])).all(dim=1)]
            if idx.numel():
                out[d] = idx.contiguous()
    return out


class BorderExchange:
    def __init__(self, boxes_lo, boxes_hi, model2rank, rank: int, world: int, device, group=None,
                 refresh_interval: int = 1, enabled: bool = True):
        self.lo = torch.as_tensor(boxes_lo, dtype=torch.float32, device=device)
        self.hi = torch.as_tensor(boxes_hi, dtype=torch.float32, device=device)
        self.model2rank = list(model2rank)
        self.M = len(self.model2rank)
        self.rank, self.world, self.device, self.group = rank, world, torch.device(device), group
        self.refresh_interval = max(1, refresh_interval)
        # a selection that is kept for several steps is made with a slightly larger extent, so that a Gaussian that
        # starts to reach a neighbour during the interval is lent already (a superset is harmless: the half-Gaussian
        # clip decides per pixel what counts)
        self.margin = 0.05 if self.refresh_interval > 1 else 0.0
        self.enabled = enabled
        self._step = 0
        self._index: dict[tuple[int, int], torch.Tensor] = {}   # (src local model, dst model) -> row ids
        self._counts = None                                     # (M,M) rows lent by src to dst
        self._rows: dict[int, torch.Tensor] = {}                # dst local model -> (n,59) borrowed rows
        self._grads: dict[int, torch.Tensor] = {}               # dst local model -> (n,60) their gradients
        self._layout: dict[int, list[tuple[int, int]]] = {}     # dst -> [(src, n)] in src order
        self._views: dict[int, dict] = {}
        self._need_grads = False

    def invalidate(self):
        """Forget the cached selection (after densification, pruning, repartition or a checkpoint load)."""
        self._index.clear()
        self._counts = None
        self._step = 0

    # -- selection ------------------------------------------------------------------------------
    def _select(self, stores: dict[int, GaussianStore]):
        counts = torch.zeros(self.M, self.M, dtype=torch.int64, device=self.device)
        self._index.clear()
        for m, st in stores.items():
            if st.count == 0:
                continue
            for d, idx in select_border(st, m, self.lo, self.hi, self.margin).items():
                self._index[(m, d)] = idx
                counts[m, d] = idx.numel()
        if self.world > 1:
            dist.all_reduce(counts, group=self.group)
        self._counts = counts.cpu()

    # -- forward exchange ---------------------------------------------------------------------------
    def refresh(self, stores: dict[int, GaussianStore], need_grads: bool):
        """Gather the lent rows and deliver them to the borrowing sub-models (local copy or P2P)."""
        if not self.enabled or self.M == 1:
            return
        if self._counts is None or self._step % self.refresh_interval == 0:
            self._select(stores)
        self._step += 1
        self._need_grads = need_grads
        ops, send_keep = [], []
        self._layout = {d: [] for d in stores}
        for d in stores:
            total = int(self._counts[:, d].sum())
            buf = self._rows.get(d)
            if buf is None or buf.shape[0] != total:
                buf = torch.empty(total, RECORD, dtype=torch.float32, device=self.device)
                self._rows[d] = buf
                self._grads[d] = torch.zeros(total, GRAD_COLS, dtype=torch.float32, device=self.device)
                self._views.pop(d, None)
        # sends: (src local, dst remote) ; receives: (src remote, dst local); same (src,dst) order on both sides
        for s in range(self.M):
            for d in range(self.M):
                n = int(self._counts[s, d])
                if n == 0 or s == d:
                    continue
                rs, rd = self.model2rank[s], self.model2rank[d]
                if rd == self.rank:
                    off = sum(k for _, k in self._layout[d])
                    dst_rows = self._rows[d][off:off + n]
                    self._layout[d].append((s, n))
                    if rs == self.rank:
                        dst_rows.copy_(stores[s].records("params", self._index[(s, d)]))
                    else:
                        ops.append(dist.P2POp(dist.irecv, dst_rows, rs, self.group))
                elif rs == self.rank:
                    rows = stores[s].records("params", self._index[(s, d)]).contiguous()
                    send_keep.append(rows)
                    ops.append(dist.P2POp(dist.isend, rows, rd, self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        if need_grads:
            for g in self._grads.values():
                g.zero_()

    def segment(self, d: int, with_grads: bool) -> Segment | None:
        """Borrowed Gaussians of local sub-model ``d`` as a render segment (column views of the row buffer
        would be strided, so the columns are split into contiguous tensors once per refresh)."""
        if not self.enabled or self.M == 1:
            return None
        rows = self._rows.get(d)
        if rows is None or rows.shape[0] == 0:
            return None
        n = rows.shape[0]
        cols, off = {}, 0
        for name, w in zip(NAMES, WIDTHS):
            cols[name] = rows[:, off:off + w].contiguous()
            off += w
        seg = Segment(cols["xyz"], cols["sh"], cols["scale"], cols["rot"], cols["opacity"])
        if with_grads:
            g = {name: torch.zeros(n, w, dtype=torch.float32, device=self.device) for name, w in zip(NAMES, WIDTHS)}
            seg.g_xyz, seg.g_sh, seg.g_scale, seg.g_rot, seg.g_opacity = g["xyz"], g["sh"], g["scale"], g["rot"], g["opacity"]
            seg.stat_grad = torch.zeros(n, dtype=torch.float32, device=self.device)
            self._views.setdefault(d, []).append(seg)
        return seg

    # -- backward exchange --------------------------------------------------------------------------
    def return_grads(self, stores: dict[int, GaussianStore]):
        """Send the gradients of borrowed rows back and add them into the owners' gradient blocks."""
        if not self.enabled or self.M == 1 or not self._need_grads:
            return
        for d, segs in self._views.items():
            if not segs:
                continue
            total = torch.zeros_like(self._grads[d])
            for seg in segs:
                total += torch.cat([seg.g_xyz, seg.g_sh, seg.g_scale, seg.g_rot, seg.g_opacity, seg.stat_grad[:, None]], 1)
            self._grads[d] = total
        self._views = {}
        ops, recv = [], []
        for s in range(self.M):
            for d in range(self.M):
                n = int(self._counts[s, d])
                if n == 0 or s == d:
                    continue
                rs, rd = self.model2rank[s], self.model2rank[d]
                if rd == self.rank:
                    off = 0
                    for ss, k in self._layout[d]:
                        if ss == s:
                            break
                        off += k
                    g = self._grads[d][off:off + n]
                    if rs == self.rank:
                        self._accumulate(stores[s], self._index[(s, d)], g)
                    else:
                        ops.append(dist.P2POp(dist.isend, g.contiguous(), rs, self.group))
                elif rs == self.rank:
                    buf = torch.empty(n, GRAD_COLS, dtype=torch.float32, device=self.device)
                    recv.append((s, d, buf))
                    ops.append(dist.P2POp(dist.irecv, buf, rd, self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        for s, d, buf in recv:
            self._accumulate(stores[s], self._index[(s, d)], buf)

    @staticmethod
    def _accumulate(store: GaussianStore, idx: torch.Tensor, g: torch.Tensor):
        gv = store.views("grads")
        off = 0
        for name, w in zip(NAMES, WIDTHS):
            gv[name].index_add_(0, idx, g[:, off:off + w])
            off += w
        store.grad_accum[:store.count].index_add_(0, idx, g[:, off])
        store.mark_touched(idx)
