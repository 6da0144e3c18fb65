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
        with torch.cuda.device(device):
            p = ctypes.c_void_p()
            rc = lib.rgs_cuda_ipc_alloc(self.nbytes + 2 * GUARD_BYTES, ctypes.byref(p))
            if rc:
                raise RuntimeError(f"cudaMalloc of the exchange region failed ({rc})")
            self._alloc_ptr = int(p.value)
            self.local_ptr = self._alloc_ptr + GUARD_BYTES
            handle = ctypes.create_string_buffer(64)
            if self.world > 1:
                rc = lib.rgs_cuda_ipc_get_handle(self._alloc_ptr, handle)
                if rc:
                    raise RuntimeError(f"cudaIpcGetMemHandle failed ({rc})")
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self.ptrs = []
            self._peer_bases: dict[int, int] = {}
            for r in range(self.world):
                if r == self.rank:
                    self.ptrs.append(self.local_ptr)
                else:
                    q = ctypes.c_void_p()
                    rc = lib.rgs_cuda_ipc_open(handles[r], ctypes.byref(q))
                    if rc:
                        raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed ({rc})")
                    self._peer_bases[r] = int(q.value)
                    self.ptrs.append(int(q.value) + GUARD_BYTES)
        self._whole = torch.as_tensor(_DevBuf(self._alloc_ptr, self.nbytes + 2 * GUARD_BYTES), device=device)
        self._guards = (self._whole[:GUARD_BYTES].view(torch.int32), self._whole[GUARD_BYTES + self.nbytes:].view(torch.int32))
        for gz in self._guards:
            gz.fill_(CANARY)
        self.local = self._whole[GUARD_BYTES:GUARD_BYTES + self.nbytes]
        if self.world > 1:
            dist.barrier(group)

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

    FLAG_BYTES = 256

    def __init__(self, device, group=None, max_views: int = 4, region: PeerRegion | None = None):
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.max_views = max_views
        self.region = region
        self.epoch = 0
        self.layout = None
        self.status = torch.zeros(native.CNT_WORDS, dtype=torch.int32, device=self.device)

    # -- layout -----------------------------------------------------------------------------------
    def _ensure(self, H: int, W: int, n_models: int, local_models: list[int], n_views: int):
        key = (H, W, n_models, tuple(local_models), max(n_views, self.max_views))
        if self.layout is not None and self.layout["key"] == key:
            return
        if self.region is not None:
            self.region.close()
        V = key[4]
        bands = band_rows(H, self.world)
        ext = [extended(b, H) for b in bands]
        max_ext = max(e[1] - e[0] for e in ext)
        slot_bytes = max_ext * W * 16
        grad_bytes = H * W * 16
        max_local = -(-n_models // self.world)
        off_slots = self.FLAG_BYTES
        off_grads = off_slots + V * n_models * slot_bytes
        total = off_grads + V * max_local * grad_bytes
        self.region = PeerRegion(total, self.device, self.group)
        self.layout = dict(key=key, V=V, bands=bands, ext=ext, slot_bytes=slot_bytes, grad_bytes=grad_bytes,
                           off_slots=off_slots, off_grads=off_grads, n_models=n_models, H=H, W=W)
        self.flags = self.region.view(0, (self.FLAG_BYTES // 4,), torch.int32)
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*self.region.ptrs)
        self.epoch = 0

    def _slot_off(self, view: int, model: int) -> int:
        L = self.layout
        return L["off_slots"] + (view * L["n_models"] + model) * L["slot_bytes"]

    def _grad_off(self, view: int, model: int) -> int:
        L = self.layout
        return L["off_grads"] + (view * (-(-L["n_models"] // self.world)) + model // self.world) * L["grad_bytes"]

    def prepare(self, plans: list[ViewPlan], n_models: int, model2rank: list[int]):
        p0 = plans[0]
        local = [m for m in range(n_models) if model2rank[m] == self.rank]
        self._ensure(p0.H, p0.W, n_models, local, len(plans))

    # -- signalling -------------------------------------------------------------------------------
    def _signal_wait(self):
        self.epoch += 1
        native.call("p2p_signal", self.device, self._flag_ptrs, self.world, self.rank, self.epoch, sig="piiip")
        native.call("p2p_wait", self.device, self.flags, self.world, self.epoch, WAIT_BUDGET_CYCLES, self.status,
                    sig="piiipp")

    def barrier(self):
        if self.layout is not None:
            self._signal_wait()

    def check(self):
        """Host check of the wait status (call after a synchronise)."""
        st = int(self.status[0].item())
        if st:
            raise RuntimeError(f"peer wait expired: no signal from rank {st & 0xff} within the cycle budget")
        if self.region is not None and not self.region.verify_canaries():
            raise RuntimeError("a kernel stored outside the bounds of this rank's exchange region (canary overwritten)")

    # -- transport interface ------------------------------------------------------------------------
    def push_plan(self, plan: ViewPlan, model: int):
        """Rows and slot addresses for the blend epilogue of (view, model)."""
        L = self.layout
        rows0, rows1, dst = [], [], []
        for o in range(self.world):
            e = L["ext"][o]
            if e[1] > e[0]:
                rows0.append(e[0]); rows1.append(e[1])
                dst.append(self.region.ptrs[o] + self._slot_off(plan.view, model))
        n = len(dst)
        return n, (ctypes.c_int32 * max(n, 1))(*rows0), (ctypes.c_int32 * max(n, 1))(*rows1), \
            (ctypes.c_void_p * max(n, 1))(*dst)

    def exchange_partials(self, plans, local_out):
        """The pushes already happened inside the blend kernels; order them and hand out the slots as
        full-height virtual base addresses."""
        self._signal_wait()
        L = self.layout
        e = L["ext"][self.rank]
        out = {}
        for p in plans:
            out[p.view] = [self.region.ptrs[self.rank] + self._slot_off(p.view, m) - e[0] * p.W * 16 for m in p.models]
        return out

    def local_grad_images(self, plans) -> dict:
        """Gradient images of this rank's renders, inside the exchange region (peer-writable)."""
        L = self.layout
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
