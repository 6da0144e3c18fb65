"""Border-Gaussian exchange over peer-mapped memory (the fused counterpart of ``parallel/border.py``).

Same contract as :class:`BorderExchange` (``refresh`` / ``segment`` / ``return_grads`` / ``invalidate``), but no
NCCL call and no host synchronisation sits in a normal step:

* every ``refresh_interval`` steps (and after densification / repartition) the ranks recompute which Gaussians
  each sub-model lends to which neighbour, agree on the counts with one all-reduce and size the symmetric
  exchange region; between refreshes the index lists are reused.  The cached selection is made with a slightly
  enlarged extent (``margin``), so that a Gaussian that would start to qualify during the interval is already
  part of it; lending a superset is harmless because the half-Gaussian clip decides per pixel what counts;
* each step a pack kernel gathers the lent rows from the owner's column groups and stores them directly into the
  borrowing rank's render segment (``csrc/rgs_border.cu``), gradient rows travel back the same way and are added
  into the owner's gradient block; the epoch-flag barrier of the compositing transport orders producers and
  consumers.

Reference: ``result_aggregator.py:55-147`` (selection by boolean masks every iteration),
``schedulers/basic_scheduler.py:51-177`` (all-reduce of the amount matrix + batch_isend_irecv, both directions).
"""
from __future__ import annotations

import contextlib
import ctypes

import torch
import torch.distributed as dist

from ..models.gaussians import NAMES, WIDTHS, GaussianStore
from ..ops import native
from ..ops.rasterize import Segment
from .border import select_border
from .peer import PeerRegion

ROW_FLOATS = 59
GRAD_ROW_FLOATS = 60
COL_OFF = (0, 3, 51, 54, 58)  # float offsets of xyz, sh, scale, rot, opacity inside a block, per row of capacity


class PeerBorderExchange:
    def __init__(self, boxes_lo, boxes_hi, model2rank, rank: int, world: int, device, transport, group=None,
                 refresh_interval: int = 8, margin: float = 0.05):
        self.lo = torch.as_tensor(boxes_lo, dtype=torch.float32, device=device)
        self.hi = torch.as_tensor(boxes_hi, dtype=torch.float32, device=device)
        self.model2rank = list(model2rank)
        self.M = len(self.model2rank)
        self.rank, self.world, self.device, self.group = rank, world, torch.device(device), group
        self.transport = transport
        self.refresh_interval = max(1, refresh_interval)
        self.margin = margin if self.refresh_interval > 1 else 0.0
        self.enabled = True
        self.local = [m for m in range(self.M) if self.model2rank[m] == rank]
        self.slot_of, per_rank = {}, {}  # position of a model among its rank's models (any assignment)
        for m in range(self.M):
            self.slot_of[m] = per_rank.get(self.model2rank[m], 0)
            per_rank[self.model2rank[m]] = self.slot_of[m] + 1
        self.max_local = max(per_rank.values())
        self._step = 0
        self._index: dict[tuple[int, int], torch.Tensor] = {}
        self._counts = None
        self.region: PeerRegion | None = None
        self.cap_b = self.cap_r = 0
        self._segs: dict[int, Segment] = {}
        self._need_grads = False
        self._fresh = True
        self.timer = None  # a PhaseTimer of the engine: the parts of refresh / return_grads get their own entries

    def _phase(self, name: str):
        return self.timer.phase(name) if self.timer is not None and self.timer.enabled else contextlib.nullcontext()

    def invalidate(self):
        self._counts = None
        self._index.clear()
        self._step = 0

    # -- layout -------------------------------------------------------------------------------------
    def _block_bytes(self) -> int:
        return self.cap_b * ROW_FLOATS * 4

    def _ring_bytes(self) -> int:
        # gradient rows, then one "this row carries a gradient" byte per row
        return self.cap_r * GRAD_ROW_FLOATS * 4 + (self.cap_r + 255) // 256 * 256

    def _ring_flags_off(self, model: int) -> int:
        return self._ring_off(model) + self.cap_r * GRAD_ROW_FLOATS * 4

    def _block_off(self, model: int) -> int:
        return self.slot_of[model] * self._block_bytes()

    def _ring_off(self, model: int) -> int:
        return self.max_local * self._block_bytes() + self.slot_of[model] * self._ring_bytes()

    def _column_ptrs(self, base: int):
        return [base + COL_OFF[k] * self.cap_b * 4 for k in range(5)]

    # -- selection (collective) -----------------------------------------------------------------------
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
        need_b = int(self._counts.sum(0).max())
        need_r = int(self._counts.sum(1).max())
        if need_b > self.cap_b or need_r > self.cap_r or self.region is None:
            if self.region is not None:
                self.region.close()
            self.cap_b = max(4, (int(need_b * 1.25) + 3) // 4 * 4)
            self.cap_r = max(4, (int(need_r * 1.25) + 3) // 4 * 4)
            self.region = PeerRegion(self.max_local * (self._block_bytes() + self._ring_bytes()), self.device, self.group)
        c = self._counts
        self._in_off = {(s, d): int(c[:s, d].sum()) for s in range(self.M) for d in range(self.M)}    # row of s inside d's block
        self._out_off = {(s, d): int(c[s, :d].sum()) for s in range(self.M) for d in range(self.M)}   # row of d inside s's ring
        self._segs.clear()
        for d in self.local:
            n = int(c[:, d].sum())
            if n == 0:
                continue
            base = self._block_off(d)
            cols = [self.region.view(base + COL_OFF[k] * self.cap_b * 4, (n, WIDTHS[k])) for k in range(5)]
            seg = Segment(*cols)
            g = [torch.zeros(n, w, dtype=torch.float32, device=self.device) for w in WIDTHS]
            seg.g_xyz, seg.g_sh, seg.g_scale, seg.g_rot, seg.g_opacity = g
            seg.stat_grad = torch.zeros(n, dtype=torch.float32, device=self.device)
            # first gradient of a step is stored, later ones are added; the marks are cleared when the rows are pushed back
            seg.touched = torch.zeros(n, dtype=torch.uint8, device=self.device)
            self._segs[d] = seg
        self._fresh = True  # the next refresh packs every lent row, later ones only rows that may have moved

    # -- per step -------------------------------------------------------------------------------------
    def refresh(self, stores: dict[int, GaussianStore], need_grads: bool):
        if self.M == 1:
            return
        if self._counts is None or self._step % self.refresh_interval == 0:
            with self._phase("border.select"):
                self.transport.barrier()  # nobody still reads the old layout
                self._select(stores)
        self._step += 1
        self._need_grads = need_grads
        c = self._counts
        with self._phase("border.pack"):
            self._pack(stores, c)
        self._fresh = False
        with self._phase("border.barrier"):
            self.transport.barrier()  # rows have landed before anyone renders them

    def _pack(self, stores, c):
        for s in self.local:
            st = stores[s]
            p = st.views()
            src = (ctypes.c_void_p * 5)(*[p[name].data_ptr() for name in NAMES])
            for d in range(self.M):
                n = int(c[s, d])
                if n == 0:
                    continue
                base = self.region.ptrs[self.model2rank[d]] + self._block_off(d)
                dst = (ctypes.c_void_p * 5)(*self._column_ptrs(base))
                # between two selections only rows with Adam moments can have moved: the others are skipped
                native.call("border_pack", self.device, src, self._index[(s, d)], n, dst, self._in_off[(s, d)],
                            None if self._fresh else st.active, sig="ppipipp")

    def segment(self, d: int, with_grads: bool) -> Segment | None:
        if self.M == 1:
            return None
        return self._segs.get(d)

    def return_grads(self, stores: dict[int, GaussianStore]):
        if self.M == 1 or not self._need_grads:
            return
        c = self._counts
        with self._phase("border.push"):
            self._push_grads(c)
        with self._phase("border.barrier"):
            self.transport.barrier()  # gradient rows have landed at their owners
        with self._phase("border.add"):
            self._add_grads(stores, c)

    def _push_grads(self, c):
        for d in self.local:
            seg = self._segs.get(d)
            if seg is None:
                continue
            g = (ctypes.c_void_p * 5)(seg.g_xyz.data_ptr(), seg.g_sh.data_ptr(), seg.g_scale.data_ptr(), seg.g_rot.data_ptr(),
                                      seg.g_opacity.data_ptr())
            for s in range(self.M):
                n = int(c[s, d])
                if n == 0:
                    continue
                base = self.region.ptrs[self.model2rank[s]]
                rows = base + self._ring_off(s) + self._out_off[(s, d)] * GRAD_ROW_FLOATS * 4
                flags = base + self._ring_flags_off(s) + self._out_off[(s, d)]
                native.call("border_grad_push", self.device, g, seg.stat_grad, seg.touched, self._in_off[(s, d)], n, rows, flags,
                            sig="pppiippp")

    def _add_grads(self, stores, c):
        for s in self.local:
            st = stores[s]
            gv = st.views("grads")
            g = (ctypes.c_void_p * 5)(*[gv[name].data_ptr() for name in NAMES])
            for d in range(self.M):
                n = int(c[s, d])
                if n == 0:
                    continue
                rows = self.region.ptrs[self.rank] + self._ring_off(s) + self._out_off[(s, d)] * GRAD_ROW_FLOATS * 4
                flags = self.region.ptrs[self.rank] + self._ring_flags_off(s) + self._out_off[(s, d)]
                native.call("border_grad_add", self.device, rows, flags, self._index[(s, d)], n, g, st.grad_accum, st.touched,
                            sig="pppipppp")

    def close(self):
        if self.region is not None:
            self.region.close()
            self.region = None
