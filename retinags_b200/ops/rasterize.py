"""Render tasks: one (camera, sub-model) rasterisation through the native kernels.

``RenderTask`` owns every buffer of one render (compacted splat records, sorted instance list,
tile ranges, per-pixel contributor counts, splat gradients) so that nothing is allocated inside
the step once capacities have settled; the reference allocates outputs plus three byte buffers on
every call (``rasterize_points.cu:71-83``) and blocks the host on the instance count
(``rasterizer_impl.cu:286-287``).  Capacities are high-water marks: the kernels count what they
*would* have needed and raise an overflow word instead of writing out of bounds; the host reads
the counters when it next synchronises anyway and grows the buffers.

``rasterize_gaussians`` is the autograd entry point with the argument list of the reference's
``GaussianRasterizer.forward`` (``diff_gaussian_rasterization_half_gaussian/__init__.py:199-232``):
activated means/scales/rotations/opacities/SHs in, premultiplied colour, depth and alpha out.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from ..data.cameras import Camera
from . import native
from .native import CNT_INST, CNT_INST2, CNT_OVERFLOW, CNT_STATUS, CNT_VIS, CNT_WORDS, RgsCamera, RgsSegment

TILE = 16
MAX_SLAB_TILES = 1 << 24  # tile keys of the two-slab path are sorted in up to three 8-bit passes
INF = float("inf")


def make_camera(cam: Camera, sh_degree: int, box_lo=None, box_hi=None, raw_params: bool = True,
                tight_rect: bool | int = True, scale_modifier: float = 1.0, bg=(0.0, 0.0, 0.0)) -> RgsCamera:
    """Fill the by-value camera/sub-model descriptor the kernels take."""
    c = RgsCamera()
    c.view[:] = cam.world_view_transform.reshape(-1).tolist()
    c.proj[:] = cam.full_proj_transform.reshape(-1).tolist()
    c.c2w[:] = cam.view_world_transform.reshape(-1).tolist()
    c.campos[:] = cam.camera_center.tolist()
    c.tan_fovx, c.tan_fovy = cam.tan_fovx, cam.tan_fovy
    c.focal_x = cam.width / (2.0 * cam.tan_fovx)
    c.focal_y = cam.height / (2.0 * cam.tan_fovy)
    c.W, c.H = cam.width, cam.height
    c.tiles_x = (cam.width + TILE - 1) // TILE
    c.tiles_y = (cam.height + TILE - 1) // TILE
    lo = [-INF] * 3 if box_lo is None else [float(v) for v in box_lo]
    hi = [INF] * 3 if box_hi is None else [float(v) for v in box_hi]
    c.box_lo[:] = lo
    c.box_hi[:] = hi
    c.bg[:] = [float(v) for v in bg]
    c.sh_degree = int(sh_degree)
    c.scale_modifier = float(scale_modifier)
    c.raw_params = 1 if raw_params else 0
    c.tight_rect = int(tight_rect)  # 0 off, 1 opacity-aware rectangle, 2 rectangle + per-tile test
    return c


@dataclass
class Segment:
    """A block of Gaussians read by a render (own or borrowed), with optional gradient sinks."""

    xyz: torch.Tensor
    sh: torch.Tensor
    scale: torch.Tensor
    rot: torch.Tensor
    opacity: torch.Tensor
    g_xyz: torch.Tensor | None = None
    g_sh: torch.Tensor | None = None
    g_scale: torch.Tensor | None = None
    g_rot: torch.Tensor | None = None
    g_opacity: torch.Tensor | None = None
    g_mean2d: torch.Tensor | None = None
    stat_grad: torch.Tensor | None = None
    stat_denom: torch.Tensor | None = None
    stat_maxrad: torch.Tensor | None = None
    touched: torch.Tensor | None = None  # uint8 (count): see RgsSegment.touched

    @property
    def count(self) -> int:
        return int(self.xyz.shape[0])

    def struct(self, with_grads: bool = True) -> RgsSegment:
        s = RgsSegment()
        for name in ("xyz", "sh", "scale", "rot", "opacity"):
            t = getattr(self, name)
            assert t.is_contiguous() and t.dtype == torch.float32, name
            setattr(s, name, t.data_ptr())
        for name in ("g_xyz", "g_sh", "g_scale", "g_rot", "g_opacity", "g_mean2d", "stat_grad", "stat_denom",
                     "stat_maxrad"):
            t = getattr(self, name) if with_grads else None
            if t is not None:
                assert t.is_contiguous() and t.dtype == torch.float32, name
            setattr(s, name, None if t is None else t.data_ptr())
        tt = self.touched if with_grads else None
        if tt is not None:
            assert tt.is_contiguous() and tt.dtype == torch.uint8
        s.touched = None if tt is None else tt.data_ptr()
        s.count = self.count
        return s


class SortScratch:
    """Ping-pong buffers and histogram scratch of the radix sort, shared by all tasks of a device."""

    def __init__(self, device: torch.device):
        self.device = device
        self.cap = 0
        self.keys_tmp = self.vals_tmp = self.words = None

    def ensure(self, cap_inst: int):
        if cap_inst <= self.cap:
            return
        kind = "cuda" if self.device.type == "cuda" else "cpu"
        fn = getattr(native.lib(kind), f"rgs_{kind}_sort_scratch_words")
        fn.argtypes = [ctypes.c_int64]
        fn.restype = ctypes.c_int64
        words = int(fn(cap_inst))
        self.keys_tmp = torch.empty(cap_inst, dtype=torch.int64, device=self.device)
        self.vals_tmp = torch.empty(cap_inst, dtype=torch.int32, device=self.device)
        self.words = torch.empty(words, dtype=torch.int32, device=self.device)
        self.cap = cap_inst


class BinScratch:
    """Transient buffers of the depth-ordered binning (rgs_binning.cu), shared by all tasks of a device."""

    def __init__(self, device: torch.device):
        self.device = device
        self.cap_vis = self.cap_inst = 0
        self.words_n = 0

    def ensure(self, cap_vis: int, cap_inst: int):
        dev = self.device
        grown = False
        if cap_vis > self.cap_vis:
            self.cap_vis = cap_vis
            self.slot_depth = torch.empty(cap_vis, dtype=torch.int32, device=dev)
            self.slot_rect = torch.empty(cap_vis, dtype=torch.int64, device=dev)
            self.slot_cnt = torch.empty(cap_vis, dtype=torch.int32, device=dev)
            self.vis = [torch.empty(cap_vis, dtype=torch.int32, device=dev) for _ in range(4)]
            grown = True
        if cap_inst > self.cap_inst:
            self.cap_inst = cap_inst
            self.inst_keys = torch.empty(cap_inst, dtype=torch.int32, device=dev)
            self.inst_keys_tmp = torch.empty(cap_inst, dtype=torch.int32, device=dev)
            self.inst_vals_tmp = torch.empty(cap_inst, dtype=torch.int32, device=dev)
            grown = True
        if grown:
            kind = "cuda" if dev.type == "cuda" else "cpu"
            fn = getattr(native.lib(kind), f"rgs_{kind}_bin_scratch_words")
            fn.argtypes = [ctypes.c_int64, ctypes.c_int64]
            fn.restype = ctypes.c_int64
            self.words = torch.empty(int(fn(self.cap_vis, self.cap_inst)), dtype=torch.int32, device=dev)


_SCRATCH: dict[str, SortScratch] = {}
_BIN_SCRATCH: dict[str, BinScratch] = {}


def bin_scratch(device: torch.device) -> BinScratch:
    key = str(device)
    if key not in _BIN_SCRATCH:
        _BIN_SCRATCH[key] = BinScratch(device)
    return _BIN_SCRATCH[key]


def release_scratch():
    """Drop the shared sort/binning buffers (they are re-created on demand)."""
    _SCRATCH.clear()
    _BIN_SCRATCH.clear()


def sort_scratch(device: torch.device) -> SortScratch:
    key = str(device)
    if key not in _SCRATCH:
        _SCRATCH[key] = SortScratch(device)
    return _SCRATCH[key]


class RenderTask:
    """State of one rasterisation, kept between forward and backward."""

    def __init__(self, device, inst_per_gaussian: float = 4.0, min_inst: int = 1 << 16, binning: str = "depth_first"):
        self.device = torch.device(device)
        # "depth_first": sort visible splats by depth, emit in order, 2-pass tile sort (rgs_binning.cu);
        # "keyed": emit 64-bit (tile|depth) keys and sort them in 6 passes (rgs_raster.cu + rgs_sort.cu)
        self.binning = binning
        self.inst_per_gaussian = inst_per_gaussian
        self.min_inst = min_inst
        self.cap_vis = 0
        self.cap_inst = 0
        self.hw = (0, 0)
        self.cam: RgsCamera | None = None
        self.counters = torch.zeros(CNT_WORDS, dtype=torch.int32, device=self.device)
        # overflow flag and status word of every forward since the last poll (the counters restart with each forward)
        self._sticky = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._host_sticky = torch.zeros(2, dtype=torch.int32)
        self._host_counters = torch.zeros(CNT_WORDS, dtype=torch.int32)
        if self.device.type == "cuda":
            self._host_counters = self._host_counters.pin_memory()
            self._host_sticky = self._host_sticky.pin_memory()
        self._event = None
        self.splats = self.vis_ids = self.aux = self.keys = self.vals = self.ranges = None
        self.out = self.depth = self.n_contrib = self.splat_grads = None
        self.total_count = 0
        self.timer = None  # optional utils.profiler.PhaseTimer for per-kernel-group timing
        # Two-slab forward (CUDA, depth-first binning): bin and blend the nearest splats first, then emit instances of
        # the rest only for tiles that are not saturated yet. Bit-identical output, fewer instances in dense scenes.
        self.slabs = os.environ.get("RGS_SLABS", "1") == "1"
        # share of the depth-ordered splats in the near slab, /256. Small is right: the near slab only has to finish the
        # tiles that saturate early, and every splat it holds is binned without the finished-tile filter (measured at
        # 62.9 M Gaussians, one GPU: 12.2 ms per step with 32/256, 10.6 with 6/256, 10.5 with 4/256; 2/256 overflowed)
        self.slab_frac256 = int(os.environ.get("RGS_SLAB_FRACTION", "6"))
        self._pending_cap = 0             # capacity that poll() asked for; applied by the next forward
        self._need_a = self._need_b = 0   # largest instance counts of the near / far slab seen so far
        self._need_known = False
        self._slab_active = False    # the last forward used two slabs (the backward walks two lists)
        self._base_b = 0
        self.ranges_b = self.tile_done = self.sat = None
        self._own_order = self._own_rect = None  # set by forward_near: depth order / tile rectangles kept by the task
        self._want_depth = False
        self._seg_structs = None  # ctypes array of the segments of the current forward (kept alive for the colour passes)
        # debug mode: accumulate the blend backward through 64-bit fixed point so that two runs give identical bits
        self.deterministic = os.environ.get("RGS_DETERMINISTIC", "0") == "1"
        self._fixed_acc = None

    def _phase(self, name: str):
        import contextlib
        return self.timer.phase(name) if self.timer is not None else contextlib.nullcontext()

    # -- buffers ------------------------------------------------------------------------------
    def _ensure(self, n_gauss: int, H: int, W: int, want_depth: bool):
        dev = self.device
        if n_gauss > self.cap_vis:
            self.cap_vis = max(int(n_gauss), 1)
            self.splats = torch.empty(self.cap_vis, native.SPLAT_FLOATS, dtype=torch.float32, device=dev)
            self.vis_ids = torch.empty(self.cap_vis, dtype=torch.int32, device=dev)
            self.aux = torch.empty(self.cap_vis, dtype=torch.int32, device=dev)
            self.splat_grads = torch.empty(self.cap_vis, native.SPLAT_FLOATS, dtype=torch.float32, device=dev)
        want_inst = max(int(n_gauss * self.inst_per_gaussian), self.min_inst)
        if self.cap_inst == 0:
            self._grow_inst(want_inst)
        if (H, W) != self.hw:
            self.hw = (H, W)
            tiles = ((H + TILE - 1) // TILE) * ((W + TILE - 1) // TILE)
            self.ranges = torch.zeros(tiles, 2, dtype=torch.int32, device=dev)
            self.ranges_b = torch.zeros(tiles, 2, dtype=torch.int32, device=dev)
            self.tile_done = torch.zeros(tiles, dtype=torch.uint8, device=dev)
            self.sat = torch.zeros(((H + TILE - 1) // TILE + 1) * ((W + TILE - 1) // TILE + 1), dtype=torch.int32, device=dev)
            self.out = torch.empty(H, W, 4, dtype=torch.float32, device=dev)
            self.n_contrib = torch.empty(H, W, dtype=torch.int32, device=dev)
            self.depth = None
        if want_depth and self.depth is None:
            self.depth = torch.empty(H, W, dtype=torch.float32, device=dev)

    def _grow_inst(self, cap: int):
        cap = int(min(max(cap, self.min_inst, 64), 0xFFFFFF00))
        self.cap_inst = cap
        self.vals = torch.empty(cap, dtype=torch.int32, device=self.device)
        if self.binning == "keyed":
            self.keys = torch.empty(cap, dtype=torch.int64, device=self.device)
            sort_scratch(self.device).ensure(cap)

    # -- forward ------------------------------------------------------------------------------
    def forward(self, cam: RgsCamera, segments: list[Segment], want_depth: bool = False, out: torch.Tensor | None = None,
                check: bool = False, push=None) -> torch.Tensor:
        """Rasterise ``segments`` for ``cam``; returns the (H,W,4) premultiplied RGB + T image.

        ``out`` lets the caller provide the destination; ``push`` = (n, row0[], row1[], dst[]) makes the
        blend epilogue also store row ranges into compositing slots (local or peer-mapped).  With ``check`` the counters are read back (host sync) and the render is repeated
        with larger buffers when the instance capacity was exceeded.
        """
        H, W = cam.H, cam.W
        self.cam = cam
        self.total_count = sum(s.count for s in segments)
        self._ensure(self.total_count, H, W, want_depth)
        for attempt in range(12):
            if self._pending_cap > self.cap_inst:  # asked for by poll() or by the previous attempt
                self._grow_inst(self._pending_cap)
            self._pending_cap = 0
            dst = self.out if out is None else out
            self.counters.zero_()
            base = 0
            if self.binning == "keyed":
                for seg in segments:
                    if seg.count:
                        native.call("project_emit", self.device, cam, seg.struct(False), base, self.splats, self.vis_ids,
                                    self.aux, self.cap_vis, self.keys, self.vals, self.cap_inst, self.counters,
                                    self.splat_grads)
                    base += seg.count
                sc = sort_scratch(self.device)
                sc.ensure(self.cap_inst)
                native.call("sort_ranges", self.device, self.keys, self.vals, sc.keys_tmp, sc.vals_tmp, self.cap_inst,
                            self.counters, cam.tiles_x * cam.tiles_y, self.ranges, sc.words)
            else:
                bs = bin_scratch(self.device)
                bs.ensure(self.cap_vis, self.cap_inst)
                self._own_order = self._own_rect = None
                # two-phase projection: conservative cull of everything, full projection of the survivors;
                # the candidate list reuses a ping-pong buffer of the depth sort (free until then)
                structs = (RgsSegment * len(segments))(*[s.struct(False) for s in segments])
                tiles = cam.tiles_x * cam.tiles_y
                self._slab_active = self.slabs and cam.tight_rect < 2 and 8 <= tiles <= MAX_SLAB_TILES
                self._seg_structs = (structs, len(segments), segments)
                with self._phase("fwd.project"):
                    # with two slabs the SH colours are evaluated later, only for splats that get tile instances
                    native.call("project_slots2_geom" if self._slab_active else "project_slots2", self.device, cam, structs,
                                len(segments), bs.vis[3], self.cap_vis, self.splats, self.vis_ids, self.aux, self.cap_vis,
                                bs.slot_depth, bs.slot_rect, bs.slot_cnt, self.counters, self.splat_grads,
                                sig=native.SIGNATURES["project_slots2"])
                if self._slab_active:
                    self._forward_slabs(cam, bs, dst, want_depth, push)
                    self.last_out = dst
                    if not check:
                        self._record_counters()
                        return dst
                    cnt = self.counters.tolist()
                    if cnt[CNT_STATUS]:
                        raise RuntimeError(f"rasteriser status {cnt[CNT_STATUS]}")
                    self._note_slab_counts(cnt[CNT_INST] & 0xFFFFFFFF, cnt[CNT_INST2] & 0xFFFFFFFF)
                    if not cnt[CNT_OVERFLOW]:
                        self.n_vis, self.n_inst = cnt[CNT_VIS], cnt[CNT_INST] + cnt[CNT_INST2]
                        return dst
                    continue
                with self._phase("fwd.binning"):
                    native.call("bin_instances", self.device, cam, self.splats, bs.slot_depth, bs.slot_rect, bs.slot_cnt,
                                self.cap_vis, bs.vis[0],
                                bs.vis[1], bs.vis[2], bs.vis[3], bs.inst_keys, self.vals, bs.inst_keys_tmp,
                                bs.inst_vals_tmp, self.cap_inst, self.counters, cam.tiles_x, cam.tiles_y * cam.tiles_x,
                                self.ranges, bs.words)
            with self._phase("fwd.blend"):
                if push is None:
                    native.call("blend_fwd", self.device, cam, self.ranges, self.vals, self.splats, dst,
                                self.depth if want_depth else None, self.n_contrib, self.counters)
                else:  # (n, row0[], row1[], dst[]): also store the rows into the owners' compositing slots
                    native.call("blend_fwd_push", self.device, cam, self.ranges, self.vals, self.splats, dst,
                                self.depth if want_depth else None, self.n_contrib, self.counters, push[0], push[1],
                                push[2], push[3])
            self.last_out = dst
            if not check:
                self._record_counters()
                return dst
            cnt = self.counters.tolist()
            if cnt[CNT_STATUS]:
                raise RuntimeError(f"rasteriser wait expired (status {cnt[CNT_STATUS]})")
            if not cnt[CNT_OVERFLOW]:
                self.n_vis, self.n_inst = cnt[CNT_VIS], cnt[CNT_INST]
                return dst
            need = cnt[CNT_INST] & 0xFFFFFFFF
            self._grow_inst(int(need * 1.25) + 1024)
        raise RuntimeError("the instance buffers still overflow after 12 attempts to grow them")

    _SIG_BIN_SLAB = "pppp" + "i" + "pppp" + "pppp" + "ii" + "p" + "i" + "p" + "p" + "iii" + "pp" + "p"
    _SIG_FWD_SLAB = "pppppppppp" + "iii" + "ppp" + "p" + "p"
    _SIG_BWD_SLAB = "ppp" + "i" + "pppppppp" + "i" + "p" + "p"

    def _slab_regions(self):
        # The buffers are shared in proportion to the largest needs seen so far, so that both slabs keep the same head
        # room (_note_slab_counts keeps the total at 1.3x of their sum or more); before any count is known: 40 : 60.
        share = (self._need_a + 2048.0) / (self._need_a + self._need_b + 4096.0) if self._need_known else 0.4
        want_a = int(self.cap_inst * min(0.95, max(0.05, share)))
        floor = min(1024, self.cap_inst // 4)  # both regions stay inside the buffer however small it is
        cap_a = max(4, max(floor, min(want_a, self.cap_inst - floor)) // 4 * 4)
        assert 0 < cap_a < self.cap_inst
        self._base_b = cap_a
        return cap_a, self.cap_inst - cap_a

    def _bin_slab(self, cam, bs, slab, off, cap, ranges, filt):
        tiles = cam.tiles_x * cam.tiles_y
        # the depth order and the tile rectangles live in the shared scratch, or in buffers of the task when the two halves
        # of the forward are separated by other tasks' work (forward_near / forward_far)
        rect = bs.slot_rect if self._own_rect is None else self._own_rect
        order = bs.vis[1] if self._own_order is None else self._own_order
        native.call("bin_slab", self.device, cam, bs.slot_depth, rect, bs.slot_cnt, self.cap_vis, bs.vis[0], order,
                    bs.vis[2], bs.vis[3], bs.inst_keys, self.vals, bs.inst_keys_tmp, bs.inst_vals_tmp, off, cap, self.counters,
                    tiles, ranges, bs.words, self.cap_inst, slab, self.slab_frac256, filt, self.sat if filt is not None else None,
                    sig=self._SIG_BIN_SLAB)

    def _colour_slab(self, cam, bs, slab):
        """SH colours of the slab's splats that have tile instances (the projection left them at zero)."""
        order = bs.vis[1] if self._own_order is None else self._own_order
        structs, nseg, _ = self._seg_structs
        with self._phase("fwd.project"):
            native.call("colour_slab", self.device, cam, structs, nseg, order, bs.slot_cnt, self.counters, self.cap_vis,
                        self.slab_frac256, slab, self.splats, self.vis_ids, self.aux, sig="ppipppiiipppp")

    def _blend_slab(self, cam, dst, depth, mode, push, occl):
        p = push if (mode == 2 and push is not None) else (0, None, None, None)
        native.call("blend_fwd_slab", self.device, cam, self.ranges, self.ranges_b, self.vals, self.splats, dst, depth,
                    self.n_contrib, self.counters, self.tile_done, self._base_b, mode, p[0], p[1], p[2], p[3], occl,
                    sig=self._SIG_FWD_SLAB)

    def _forward_slabs_near(self, cam: RgsCamera, bs: BinScratch, dst: torch.Tensor, want_depth: bool, occl=None):
        """Near slab: bin (only tiles outside ``occl``) and blend; leaves ``tile_done`` = own finished tiles | occl."""
        cap_a, _ = self._slab_regions()
        depth = self.depth if want_depth else None
        with self._phase("fwd.binning"):
            self._bin_slab(cam, bs, 0, 0, cap_a, self.ranges, occl)
        self._colour_slab(cam, bs, 0)
        with self._phase("fwd.blend"):
            self._blend_slab(cam, dst, depth, 1, None, occl)

    def _forward_slabs_far(self, cam: RgsCamera, bs: BinScratch, dst: torch.Tensor, want_depth: bool, push, occl=None):
        """Far slab for the tiles that neither this sub-model (near slab) nor nearer sub-models (``occl``, optional:
        what became known after the near slab) have finished; ``tile_done`` ends as the final state of the tiles."""
        cap_a = self._base_b
        depth = self.depth if want_depth else None
        if occl is not None:
            native.call("tile_maps_or", self.device, native.pointer_array([occl]), 1, self.tile_done, self.tile_done.numel(), 0,
                        sig="pipiip")
        with self._phase("fwd.binning"):
            self._bin_slab(cam, bs, 1, cap_a, self.cap_inst - cap_a, self.ranges_b, self.tile_done)
        self._colour_slab(cam, bs, 1)
        with self._phase("fwd.blend"):
            self._blend_slab(cam, dst, depth, 2, push, None)

    def _forward_slabs(self, cam: RgsCamera, bs: BinScratch, dst: torch.Tensor, want_depth: bool, push):
        self._forward_slabs_near(cam, bs, dst, want_depth)
        self._forward_slabs_far(cam, bs, dst, want_depth, push)

    # -- forward in two halves: what the occlusion exchange between sub-models needs ---------------------------------
    def forward_near(self, cam: RgsCamera, segments: list[Segment], want_depth: bool = False, occl: torch.Tensor | None = None):
        """First half of an unchecked two-slab forward: projection and the near slab, skipping the tiles of ``occl``
        (uint8 per tile: finished by nearer sub-models). Afterwards ``tile_done`` holds the tiles that are finished for
        everything behind this sub-model's near slab. The depth order and the tile rectangles are kept in buffers of the
        task, so that other tasks may run before :meth:`forward_far`."""
        H, W = cam.H, cam.W
        self.cam = cam
        self.total_count = sum(s.count for s in segments)
        self._ensure(self.total_count, H, W, want_depth)
        if self._pending_cap > self.cap_inst:
            self._grow_inst(self._pending_cap)
        self._pending_cap = 0
        self._want_depth = want_depth
        self.counters.zero_()
        bs = bin_scratch(self.device)
        bs.ensure(self.cap_vis, self.cap_inst)
        tiles = cam.tiles_x * cam.tiles_y
        self._slab_active = self.binning == "depth_first" and cam.tight_rect < 2 and 8 <= tiles <= MAX_SLAB_TILES
        if not self._slab_active:
            raise RuntimeError("forward_near needs the two-slab path (depth-first binning, 8..2^24 tiles, tight_rect < 2)")
        if self._own_order is None or self._own_order.numel() < self.cap_vis:
            self._own_order = torch.empty(self.cap_vis, dtype=torch.int32, device=self.device)
            self._own_rect = torch.empty(self.cap_vis, dtype=torch.int64, device=self.device)
        structs = (RgsSegment * len(segments))(*[s.struct(False) for s in segments])
        self._seg_structs = (structs, len(segments), segments)  # the tensors must outlive the far half's colour pass
        with self._phase("fwd.project"):
            native.call("project_slots2_geom", self.device, cam, structs, len(segments), bs.vis[3], self.cap_vis,
                        self.splats, self.vis_ids, self.aux, self.cap_vis, bs.slot_depth, self._own_rect,
                        bs.slot_cnt, self.counters, self.splat_grads, sig=native.SIGNATURES["project_slots2"])
        self._forward_slabs_near(cam, bs, self.out, want_depth, occl)

    def forward_far(self, occl: torch.Tensor | None = None, push=None) -> torch.Tensor:
        """Second half: the far slab on the tiles that are still open (``occl``: tiles that nearer sub-models finished,
        as far as known by now), with the fused push of the finished partial image."""
        bs = bin_scratch(self.device)
        bs.ensure(self.cap_vis, self.cap_inst)
        self._forward_slabs_far(self.cam, bs, self.out, self._want_depth, push, occl)
        self.last_out = self.out
        self._record_counters()
        return self.out

    @staticmethod
    def can_split(cam: RgsCamera) -> bool:
        tiles = cam.tiles_x * cam.tiles_y
        return cam.tight_rect < 2 and 8 <= tiles <= MAX_SLAB_TILES

    def _note_slab_counts(self, n_a: int, n_b: int):
        """Remember the largest instance counts of both slabs and make the buffers hold 1.3x of each. The needs only grow
        and the buffers never shrink, so a render that overflowed fits after at most two more attempts (the far slab's
        count is only known once the near slab fitted)."""
        self._need_a, self._need_b = max(self._need_a, n_a), max(self._need_b, n_b)
        self._need_known = True
        want = int(1.4 * (self._need_a + self._need_b)) + 65536
        if want > self.cap_inst:
            self._pending_cap = int(2.0 * (self._need_a + self._need_b)) + 65536  # applied by the next forward attempt

    def _record_counters(self):
        torch.bitwise_or(self._sticky, self.counters[CNT_OVERFLOW:CNT_STATUS + 1], out=self._sticky)
        if self.device.type == "cuda":
            self._host_sticky.copy_(self._sticky, non_blocking=True)
            self._host_counters.copy_(self.counters, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record(torch.cuda.current_stream(self.device))
        else:
            self._host_sticky.copy_(self._sticky)
            self._host_counters.copy_(self.counters)

    def poll(self) -> dict:
        """Counters of the last unchecked forward (call after the stream was synchronised).

        Grows the instance buffers when the last render overflowed or came close; returns the
        counters so that the caller can decide to redo the step.
        """
        if self._event is not None:
            self._event.synchronize()
            self._event = None
        c = self._host_counters.tolist()
        sticky = self._host_sticky.tolist()
        self._sticky.zero_()
        n_b = (c[CNT_INST2] & 0xFFFFFFFF) if self._slab_active else 0
        # `overflow` / `status` cover every forward since the previous poll, the counts are those of the last one
        info = dict(n_vis=c[CNT_VIS], n_inst=(c[CNT_INST] & 0xFFFFFFFF) + n_b, overflow=bool(c[CNT_OVERFLOW] or sticky[0]),
                    status=c[CNT_STATUS] | sticky[1])
        if info["status"]:
            what = []
            if info["status"] & 3:
                what.append("a bounded wait on a bulk copy ran out")
            if info["status"] & 4:
                what.append("a look-back wait of the single-sweep radix sort ran out (RGS_SORT=3k selects the other sort)")
            if info["status"] & 16:
                what.append("an index read from the binning buffers was out of bounds (clamped)")
            raise RuntimeError(f"rasteriser status {info['status']}: " + "; ".join(what or ["unknown"]))
        if self._slab_active:
            self._note_slab_counts(c[CNT_INST] & 0xFFFFFFFF, n_b)
        elif info["overflow"] or info["n_inst"] > 0.6 * self.cap_inst:
            # applied by the next forward: the lists of the last render stay valid for a backward that is still to come
            self._pending_cap = max(int(info["n_inst"] * 2.0) + 1024, self.cap_inst if info["overflow"] else 0)
        return info

    # -- backward -----------------------------------------------------------------------------
    def backward(self, grad_out: torch.Tensor, segments: list[Segment], grad_depth: torch.Tensor | None = None):
        """Accumulate parameter gradients of the last forward. ``grad_out`` is (H,W,4): dL/dC, dL/dT; ``grad_depth``
        (optional, (H,W)) is the gradient of the depth output (a single-pass render only)."""
        cam = self.cam
        assert grad_out.is_contiguous() and grad_out.shape == (cam.H, cam.W, 4)
        with self._phase("bwd.blend"):
            if grad_depth is not None:
                if self.deterministic:
                    raise NotImplementedError("a depth gradient needs the float-accumulating backward")
                assert grad_depth.is_contiguous() and grad_depth.shape == (cam.H, cam.W) and grad_depth.dtype == torch.float32
            if grad_depth is not None and not self._slab_active:
                native.call("blend_bwd_depth", self.device, cam, self.ranges, self.vals, self.splats, self.last_out,
                            self.n_contrib, grad_out, grad_depth, self.splat_grads, self.counters)
            elif self._slab_active:
                fixed = None
                if self.deterministic:
                    if self._fixed_acc is None or self._fixed_acc.numel() < 9 * self.cap_vis:
                        self._fixed_acc = torch.zeros(9 * self.cap_vis, dtype=torch.int64, device=self.device)
                    fixed = self._fixed_acc
                native.call("blend_bwd_slab", self.device, cam, self.ranges, self.ranges_b, self._base_b, self.vals, self.splats,
                            self.last_out, self.n_contrib, grad_out, self.splat_grads, self.counters, fixed, self.cap_vis,
                            grad_depth, sig=self._SIG_BWD_SLAB)
            elif self.deterministic:
                if self._fixed_acc is None or self._fixed_acc.numel() < 9 * self.cap_vis:
                    self._fixed_acc = torch.zeros(9 * self.cap_vis, dtype=torch.int64, device=self.device)
                native.call("blend_bwd_fixed", self.device, cam, self.ranges, self.vals, self.splats, self.last_out,
                            self.n_contrib, grad_out, self.splat_grads, self.counters, self._fixed_acc, self.cap_vis,
                            sig="ppppppppppip")
            else:
                native.call("blend_bwd", self.device, cam, self.ranges, self.vals, self.splats, self.last_out, self.n_contrib,
                            grad_out, self.splat_grads, self.counters)
        structs = (RgsSegment * len(segments))(*[s.struct(True) for s in segments])
        with self._phase("bwd.geometry"):
            native.call("geom_bwd", self.device, cam, structs, len(segments), self.counters, self.splats, self.vis_ids,
                        self.aux, self.splat_grads, self.cap_vis)

    def radii(self, segment_index: int, segments: list[Segment]) -> torch.Tensor:
        base = sum(s.count for s in segments[:segment_index])
        cnt = segments[segment_index].count
        r = torch.zeros(cnt, dtype=torch.int32, device=self.device)
        native.call("scatter_radii", self.device, self.counters, self.vis_ids, self.aux, base, cnt, r)
        return r


# ---------------------------------------------------------------------------------------------
# autograd entry point with the reference's interface
# ---------------------------------------------------------------------------------------------
@dataclass
class GaussianRasterizationSettings:
    """Field-for-field equivalent of the reference's settings tuple
    (``diff_gaussian_rasterization_half_gaussian/__init__.py:166-181``)."""

    image_height: int
    image_width: int
    tanfovx: float
    tanfovy: float
    bg: torch.Tensor
    scale_modifier: float
    viewmatrix: torch.Tensor
    projmatrix: torch.Tensor
    projmatrix_inv: torch.Tensor  # view->world, transposed storage
    range_low: torch.Tensor
    range_up: torch.Tensor
    sh_degree: int
    campos: torch.Tensor
    prefiltered: bool = False
    debug: bool = False


def _settings_camera(st: GaussianRasterizationSettings) -> RgsCamera:
    c = RgsCamera()
    c.view[:] = st.viewmatrix.detach().cpu().reshape(-1).tolist()
    c.proj[:] = st.projmatrix.detach().cpu().reshape(-1).tolist()
    c.c2w[:] = st.projmatrix_inv.detach().cpu().reshape(-1).tolist()
    c.campos[:] = st.campos.detach().cpu().reshape(-1).tolist()
    c.tan_fovx, c.tan_fovy = st.tanfovx, st.tanfovy
    c.focal_x = st.image_width / (2.0 * st.tanfovx)
    c.focal_y = st.image_height / (2.0 * st.tanfovy)
    c.W, c.H = st.image_width, st.image_height
    c.tiles_x = (st.image_width + TILE - 1) // TILE
    c.tiles_y = (st.image_height + TILE - 1) // TILE
    c.box_lo[:] = st.range_low.detach().cpu().reshape(-1).tolist()
    c.box_hi[:] = st.range_up.detach().cpu().reshape(-1).tolist()
    c.bg[:] = st.bg.detach().cpu().reshape(-1).tolist()
    c.sh_degree = st.sh_degree
    c.scale_modifier = st.scale_modifier
    c.raw_params = 0
    c.tight_rect = 1
    return c


class _Rasterize(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means3D, means2D, shs, opacities, scales, rotations, settings):
        dev = means3D.device
        cam = _settings_camera(settings)
        seg = Segment(means3D.contiguous(), shs.contiguous().view(-1, 48), scales.contiguous(), rotations.contiguous(),
                      opacities.contiguous().view(-1, 1))
        if shs.shape[1] != 16:
            full = torch.zeros(shs.shape[0], 16, 3, dtype=shs.dtype, device=dev)
            full[:, : shs.shape[1]] = shs
            seg.sh = full.view(-1, 48)
        task = RenderTask(dev)
        task.deterministic = False  # the backward of this interface may carry a depth gradient (float accumulation)
        out = task.forward(cam, [seg], want_depth=True, check=True)
        bg = settings.bg.to(dev).view(1, 1, 3)
        color = (out[..., :3] + out[..., 3:4] * bg).permute(2, 0, 1).contiguous()
        alpha = (1.0 - out[..., 3]).unsqueeze(0)
        depth = task.depth.unsqueeze(0).clone()
        radii = task.radii(0, [seg])
        ctx.task, ctx.seg, ctx.settings, ctx.n_sh = task, seg, settings, shs.shape[1]
        ctx.mark_non_differentiable(radii)
        return color, depth, alpha, radii

    @staticmethod
    def backward(ctx, g_color, g_depth, g_alpha, _g_radii):
        task, seg, st = ctx.task, ctx.seg, ctx.settings
        dev = seg.xyz.device
        H, W = st.image_height, st.image_width
        bg = st.bg.to(dev).view(3, 1, 1)
        grad = torch.zeros(H, W, 4, dtype=torch.float32, device=dev)
        if g_color is not None:
            grad[..., :3] = g_color.permute(1, 2, 0)
            grad[..., 3] = (g_color * bg).sum(0)
        if g_alpha is not None:
            grad[..., 3] -= g_alpha[0]
        n = seg.count
        seg.g_xyz = torch.zeros(n, 3, device=dev)
        seg.g_sh = torch.zeros(n, 48, device=dev)
        seg.g_scale = torch.zeros(n, 3, device=dev)
        seg.g_rot = torch.zeros(n, 4, device=dev)
        seg.g_opacity = torch.zeros(n, 1, device=dev)
        seg.g_mean2d = torch.zeros(n, 2, device=dev)
        gd = None
        if g_depth is not None and bool((g_depth != 0).any()):
            gd = g_depth[0].contiguous().float()
        task.backward(grad.contiguous(), [seg], grad_depth=gd)
        g_means2D = torch.zeros(n, 3, device=dev)
        g_means2D[:, :2] = seg.g_mean2d
        g_sh = seg.g_sh.view(n, 16, 3)[:, : ctx.n_sh]
        return seg.g_xyz, g_means2D, g_sh, seg.g_opacity, seg.g_scale, seg.g_rot, None


def rasterize_gaussians(means3D, means2D, shs, opacities, scales, rotations, settings: GaussianRasterizationSettings):
    """(color (3,H,W), depth (1,H,W), alpha (1,H,W), radii (P)) for activated inputs."""
    return _Rasterize.apply(means3D, means2D, shs, opacities, scales, rotations, settings)


class GaussianRasterizer(torch.nn.Module):
    """Module wrapper with the call signature of the reference's ``GaussianRasterizer``."""

    def __init__(self, raster_settings: GaussianRasterizationSettings):
        super().__init__()
        self.raster_settings = raster_settings

    def forward(self, means3D, means2D, opacities, shs=None, colors_precomp=None, scales=None, rotations=None,
                cov3D_precomp=None):
        if shs is None or colors_precomp is not None or cov3D_precomp is not None:
            raise NotImplementedError("only the SH + scale/rotation path exists (the one the reference's trainer uses)")
        return rasterize_gaussians(means3D, means2D, shs, opacities, scales, rotations, self.raster_settings)

    def markVisible(self, positions: torch.Tensor) -> torch.Tensor:
        """Boolean mask of the points in front of the near plane (``GaussianRasterizer.markVisible`` of the
        reference, ``diff_gaussian_rasterization_half_gaussian/__init__.py:188-197``)."""
        cam = _settings_camera(self.raster_settings)
        pts = positions.detach().float().contiguous()
        out = torch.zeros(pts.shape[0], dtype=torch.uint8, device=pts.device)
        native.call("mark_visible", pts.device, pts, pts.shape[0], cam, out, sig="pippp")
        return out.bool()
