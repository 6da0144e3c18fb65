"""Fused peer-to-peer compositing transport (one process per GPU, NVLink peer-mapped memory).

Every rank allocates one exchange region with ``cudaMalloc``, publishes its CUDA-IPC handle through
the ``torch.distributed`` control plane and maps the regions of all peers.  A region holds

* a flag array (one 32-bit epoch word per rank),
* the *slots* in which this rank, as owner of a row band, receives the partial images of every
  (view, sub-model): only the rows of its band plus one tile row of halo on each side,
* the *gradient images* of the sub-models this rank renders, into which the owners of the bands
  store ``dL/d(partial)``.

No copy kernel and no NCCL call moves image bytes: the blend kernel's epilogue stores each finished
pixel into the owners' slots (``rgs_cuda_blend_fwd_push``), and the compositing backward kernel takes
peer-mapped gradient images as its outputs.  Ordering is by epoch flags (``rgs_p2p.cu``): producers
signal after their kernels, consumers wait (bounded) before theirs.

Counterpart in the reference: ``parallel_utils/schedulers/basic_scheduler.py:51-123`` +
``communicate_utils/core.py:37-65`` (zip -> batch_isend_irecv -> synchronise -> unzip clones).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import native
from .compositing import ViewPlan, band_rows, extended

WAIT_BUDGET_CYCLES = 20_000_000_000  # ~10 s at 2 GHz; the wait gives up and reports after that


class _DevBuf:
    """Expose raw device memory to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


GUARD_BYTES = 256           # canary zone in front of and behind the usable bytes of a region
CANARY = 0x5A5AC3C3          # pattern of the canary words (int32)


class PeerRegion:
    """Symmetric region: the same byte size on every rank, mapped everywhere.

    The usable bytes sit between two guard zones filled with a canary pattern; ``verify_canaries`` tells whether a
    kernel (of this rank or of a peer: the region is mapped everywhere) stored outside the region's bounds."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        self.device, self.group = device, group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.nbytes = int((nbytes + 255) // 256 * 256)
        lib = native.lib("cuda")
        for fn, args in (("rgs_cuda_ipc_alloc", [ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p)]),
                         ("rgs_cuda_ipc_free", [ctypes.c_void_p]),
                         ("rgs_cuda_ipc_get_handle", [ctypes.c_void_p, ctypes.c_char_p]),
                         ("rgs_cuda_ipc_open", [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
                         ("rgs_cuda_ipc_close", [ctypes.c_void_p])):
            f = getattr(lib, fn)
            f.argtypes, f.restype = args, ctypes.c_int
        self._lib = lib
        # Every step that can fail on one rank only (allocation, export, mapping a peer's handle) is followed by an
        # exchange of the outcome, so that all ranks raise together instead of one raising while the others wait in the
        # next collective.
        self._alloc_ptr = 0
        self._peer_bases: dict[int, int] = {}
        err = ""
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            p = ctypes.c_void_p()
            rc = lib.rgs_cuda_ipc_alloc(self.nbytes + 2 * GUARD_BYTES, ctypes.byref(p))
            if rc:
                err = f"cudaMalloc of the exchange region failed ({rc})"
            else:
                self._alloc_ptr = int(p.value)
                if self.world > 1:
                    rc = lib.rgs_cuda_ipc_get_handle(self._alloc_ptr, handle)
                    if rc:
                        err = f"cudaIpcGetMemHandle failed ({rc})"
        handles = self._agree(err, bytes(handle.raw))
        self.local_ptr = self._alloc_ptr + GUARD_BYTES
        self.ptrs = []
        err = ""
        with torch.cuda.device(device):
            for r in range(self.world):
                if r == self.rank:
                    self.ptrs.append(self.local_ptr)
                    continue
                q = ctypes.c_void_p()
                rc = lib.rgs_cuda_ipc_open(handles[r], ctypes.byref(q))
                if rc:
                    err = f"cudaIpcOpenMemHandle for rank {r} failed ({rc})"
                    break
                self._peer_bases[r] = int(q.value)
                self.ptrs.append(int(q.value) + GUARD_BYTES)
        self._agree(err, None)
        self._whole = torch.as_tensor(_DevBuf(self._alloc_ptr, self.nbytes + 2 * GUARD_BYTES), device=device)
        self._guards = (self._whole[:GUARD_BYTES].view(torch.int32), self._whole[GUARD_BYTES + self.nbytes:].view(torch.int32))
        for gz in self._guards:
            gz.fill_(CANARY)
        self.local = self._whole[GUARD_BYTES:GUARD_BYTES + self.nbytes]
        if self.world > 1:
            dist.barrier(group)

    def _agree(self, err: str, payload):
        """All ranks exchange (error text, payload); when any rank failed, every rank releases what it holds and raises."""
        if self.world > 1:
            got = [None] * self.world
            dist.all_gather_object(got, (err, payload), group=self.group)
        else:
            got = [(err, payload)]
        failed = [(r, e) for r, (e, _) in enumerate(got) if e]
        if failed:
            with torch.cuda.device(self.device):
                for base in self._peer_bases.values():
                    self._lib.rgs_cuda_ipc_close(base)
                self._peer_bases.clear()
                if self._alloc_ptr:
                    self._lib.rgs_cuda_ipc_free(self._alloc_ptr)
                    self._alloc_ptr = 0
            self.ptrs = None
            raise RuntimeError("peer-mapped exchange region unavailable: " + "; ".join(f"rank {r}: {e}" for r, e in failed))
        return [pl for _, pl in got]

    def view(self, offset: int, shape, dtype=torch.float32) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        return self.local[offset:offset + nbytes].view(dtype).view(*shape)

    def verify_canaries(self) -> bool:
        """True when both guard zones still hold the pattern (synchronises the device)."""
        return all(bool((gz == CANARY).all()) for gz in self._guards)

    def close(self):
        if getattr(self, "ptrs", None) is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(self.group)
            for r in range(self.world):
                if r != self.rank:
                    self._lib.rgs_cuda_ipc_close(self._peer_bases[r])
            self.local = self._whole = self._guards = None
            self._lib.rgs_cuda_ipc_free(self._alloc_ptr)
        self.ptrs = None


class PeerTransport:
    """Compositing transport in which kernels store straight into the consumer's memory."""

    def __init__(self, device, group=None, max_views: int = 4, region: PeerRegion | None = None):
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        lib = native.lib("cuda")
        for fn in ("rgs_cuda_p2p_flag_bytes", "rgs_cuda_p2p_max_world"):
            getattr(lib, fn).restype = ctypes.c_int64
        self.FLAG_BYTES = (int(lib.rgs_cuda_p2p_flag_bytes()) + 255) // 256 * 256
        if self.world > int(lib.rgs_cuda_p2p_max_world()):
            raise RuntimeError(f"the peer transport handles at most {int(lib.rgs_cuda_p2p_max_world())} ranks "
                               f"(world size {self.world}); use the torch.distributed transport")
        self.max_views = max_views
        self.region = region
        self.epoch = 0
        self.layout = None
        self.status = torch.zeros(native.CNT_WORDS, dtype=torch.int32, device=self.device)
        self._host_status = torch.zeros(native.CNT_WORDS, dtype=torch.int32).pin_memory()
        self._status_event = None
        self.skip_word = None  # optional device counter block: its overflow word travels with every signal (attach_skip)
        # Map a small region right away: a rank whose peers are not reachable through CUDA IPC (another node, a
        # container without shared IPC namespace) fails here, on every rank together, and the caller can fall back to
        # the torch.distributed transport before any step has run.
        if region is None and self.world > 1:
            PeerRegion(4096, self.device, self.group).close()

    def attach_skip(self, counters: torch.Tensor):
        """``counters``: device int32 block (layout of the rasteriser's counters). Its overflow word is sent with every
        signal and every wait ORs the words of all ranks into it, so that all ranks drop the same optimiser step."""
        self.skip_word = counters

    # -- layout -----------------------------------------------------------------------------------
    def _ensure(self, slot_bytes: int, grad_bytes: int, n_models: int, max_local: int, n_views: int):
        V = max(n_views, self.max_views)
        L = self.layout
        if L is not None and L["n_models"] == n_models and L["max_local"] == max_local and L["V"] >= V and \
                L["slot_bytes"] >= slot_bytes and L["grad_bytes"] >= grad_bytes:
            return
        if L is not None:  # sizes only grow: a batch of smaller images reuses the region
            slot_bytes, grad_bytes, V = max(slot_bytes, L["slot_bytes"]), max(grad_bytes, L["grad_bytes"]), max(V, L["V"])
        if self.region is not None:
            self.region.close()
        off_slots = self.FLAG_BYTES
        off_grads = off_slots + V * n_models * slot_bytes
        off_maps = off_grads + V * max_local * grad_bytes
        map_bytes = (grad_bytes // (16 * 256) + 512) // 256 * 256  # one byte per 16x16 tile, with room for ragged edges
        total = off_maps + V * n_models * map_bytes
        self.region = PeerRegion(total, self.device, self.group)
        self.layout = dict(V=V, slot_bytes=slot_bytes, grad_bytes=grad_bytes, off_slots=off_slots, off_grads=off_grads,
                           n_models=n_models, max_local=max_local, off_maps=off_maps, map_bytes=map_bytes)
        self.flags = self.region.view(0, (self.FLAG_BYTES // 4,), torch.int32)
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*self.region.ptrs)
        self.epoch = 0

    def _slot_off(self, view: int, model: int) -> int:
        L = self.layout
        return L["off_slots"] + (view * L["n_models"] + model) * L["slot_bytes"]

    def _grad_off(self, view: int, model: int) -> int:
        L = self.layout
        return L["off_grads"] + (view * L["max_local"] + self._local_index[model]) * L["grad_bytes"]

    @staticmethod
    def _plan_ext(plan: ViewPlan):
        return [extended(b, plan.H) for b in plan.bands]

    def prepare(self, plans: list[ViewPlan], n_models: int, model2rank: list[int]):
        """Size the exchange region for this batch. Views may differ in size (scenes with several intrinsics): slots
        and gradient images are sized for the largest view, every view is laid out with its own width and bands."""
        per_rank: dict[int, int] = {}
        self._local_index = {}
        for m in range(n_models):  # position of a sub-model among the sub-models of its rank
            self._local_index[m] = per_rank.get(model2rank[m], 0)
            per_rank[model2rank[m]] = self._local_index[m] + 1
        slot_bytes = max(max(e[1] - e[0] for e in self._plan_ext(p)) * p.W * 16 for p in plans)
        grad_bytes = max(p.H * p.W * 16 for p in plans)
        self._ensure(slot_bytes, grad_bytes, n_models, max(per_rank.values()), len(plans))

    # -- signalling -------------------------------------------------------------------------------
    def _signal_wait(self):
        self.epoch += 1
        pay = None if self.skip_word is None else self.skip_word[native.CNT_OVERFLOW:]
        native.call("p2p_signal", self.device, self._flag_ptrs, self.world, self.rank, self.epoch, pay, sig="piiipp")
        native.call("p2p_wait", self.device, self.flags, self.world, self.epoch, WAIT_BUDGET_CYCLES, self.status, pay,
                    sig="piiippp")

    def barrier(self):
        if self.layout is not None:
            self._signal_wait()

    def record_status(self):
        """Queue a copy of the wait status to pinned host memory (no synchronisation); ``check(block=False)`` reads it
        once the copy has completed."""
        self._host_status.copy_(self.status, non_blocking=True)
        self._status_event = torch.cuda.Event()
        self._status_event.record(torch.cuda.current_stream(self.device))

    def check(self, block: bool = True):
        """Host check of the wait status and of the canaries. ``block``: synchronise and read the device words;
        otherwise only look at the last recorded copy, and only if it has arrived."""
        if block:
            st = int(self.status[0].item())
        else:
            if self._status_event is None or not self._status_event.query():
                return
            self._status_event = None
            st = int(self._host_status[0])
        if st:
            raise RuntimeError(f"peer wait expired: no signal from rank {st & 0xff} within the cycle budget")
        if block and self.region is not None and not self.region.verify_canaries():
            raise RuntimeError("a kernel stored outside the bounds of this rank's exchange region (canary overwritten)")

    # -- transport interface ------------------------------------------------------------------------
    def push_plan(self, plan: ViewPlan, model: int):
        """Rows and slot addresses for the blend epilogue of (view, model)."""
        L = self.layout
        rows0, rows1, dst = [], [], []
        for o, e in enumerate(self._plan_ext(plan)):
            if e[1] > e[0]:
                if (e[1] - e[0]) * plan.W * 16 > L["slot_bytes"]:
                    raise RuntimeError("a view needs more rows per slot than the exchange region was sized for")
                rows0.append(e[0]); rows1.append(e[1])
                dst.append(self.region.ptrs[o] + self._slot_off(plan.view, model))
        n = len(dst)
        return n, (ctypes.c_int32 * max(n, 1))(*rows0), (ctypes.c_int32 * max(n, 1))(*rows1), \
            (ctypes.c_void_p * max(n, 1))(*dst)

    def exchange_partials(self, plans, local_out):
        """The pushes already happened inside the blend kernels; order them and hand out the slots as
        full-height virtual base addresses."""
        self._signal_wait()
        out = {}
        for p in plans:
            e = self._plan_ext(p)[self.rank]
            out[p.view] = [self.region.ptrs[self.rank] + self._slot_off(p.view, m) - e[0] * p.W * 16 for m in p.models]
        return out

    def exchange_images(self, plans, local_images):
        """Move arbitrary (H,W,4) images of the local sub-models to the owners of the row bands with point-to-point
        messages of ``torch.distributed``: the off-step path (eval-time depth maps), which has no fused producer."""
        if getattr(self, "_dist_transport", None) is None:
            from .compositing import TorchDistTransport
            self._dist_transport = TorchDistTransport(self.device, self.group)
        return self._dist_transport.exchange_partials(plans, local_images)

    def exchange_done_maps(self, plans, local_maps):
        """Publish the finished-tile maps of this rank's sub-models into every peer's region (plain peer stores of a few
        KB each), order with the flag barrier, and hand out the maps of all visible sub-models: remote ones as views of
        this rank's region, local ones as given."""
        L = self.layout
        out = dict(local_maps)
        for p in plans:
            tiles = ((p.H + 15) // 16) * ((p.W + 15) // 16)
            if tiles > L["map_bytes"]:
                raise RuntimeError("a view has more tiles than the map slots of the exchange region hold")
            for m, r in zip(p.models, p.ranks):
                off = L["off_maps"] + (p.view * L["n_models"] + m) * L["map_bytes"]
                if r == self.rank:
                    dsts = [self.region.ptrs[o] + off for o in range(self.world) if o != self.rank]
                    if dsts:
                        native.call("tile_map_push", self.device, local_maps[(p.view, m)], (ctypes.c_void_p * len(dsts))(*dsts),
                                    len(dsts), tiles, sig="ppiip")
                else:
                    out[(p.view, m)] = self.region.view(off, (tiles,), torch.uint8)
        self._signal_wait()
        return out

    def local_grad_images(self, plans) -> dict:
        """Gradient images of this rank's renders, inside the exchange region (peer-writable)."""
        out = {}
        for p in plans:
            out[p.view] = {m: self.region.view(self._grad_off(p.view, m), (p.H, p.W, 4))
                           for m, r in zip(p.models, p.ranks) if r == self.rank}
        return out

    def grad_slots(self, plans, local_grad):
        """Addresses at which this owner stores dL/d(partial_k): the source rank's gradient image."""
        out = {}
        for p in plans:
            out[p.view] = [self.region.ptrs[r] + self._grad_off(p.view, m) for m, r in zip(p.models, p.ranks)]
        return out

    def return_grads(self, plans, slots, local_grad):
        self._signal_wait()

    def close(self):
        if self.region is not None:
            self.region.close()
            self.region = None
            self.layout = None
