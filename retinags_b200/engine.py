"""One training / rendering step over the sub-models hosted by this rank.

``StepEngine`` is the per-rank executor underneath the trainer: given the cameras of a batch and the
camera->sub-model relation it renders every visible local sub-model, hands the partial images to
the compositing transport, composites and evaluates the loss on the row bands this rank owns,
routes ``dL/d(partial)`` back, runs the rasteriser backward and applies one fused Adam update per
sub-model.  It corresponds to steps 1-10 of the reference's iteration
(``parallel_utils/basic_parallel_trainer/trainer4tree_partition.py:606-669``), with the six
blocking exchange phases reduced to two and no host synchronisation inside a step.
"""
from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass, field

import torch

from .data.cameras import Camera
from .models.gaussians import GaussianStore
from .ops.loss import CompositeLoss
from .ops import native
from .ops.native import CNT_OVERFLOW, CNT_WORDS
from .ops.rasterize import RenderTask, Segment, make_camera
from .parallel.compositing import LocalTransport, ViewPlan, band_rows
from .utils.profiler import PhaseTimer


@dataclass
class StepResult:
    sums: list            # per view: device tensor (3,) float64 of loss sums over this rank's band
    plans: list
    overflow: bool = False
    info: dict = field(default_factory=dict)


class StepEngine:
    def __init__(self, stores: dict[int, GaussianStore], model2rank: list[int], device, transport=None,
                 lambda_dssim: float = 0.2, background=(0.0, 0.0, 0.0), tight_rect: bool = True,
                 borrow=None):
        self.stores = stores
        self.model2rank = list(model2rank)
        self.device = torch.device(device)
        self.transport = transport if transport is not None else LocalTransport(device)
        self.rank, self.world = self.transport.rank, self.transport.world
        self.lambda_dssim = lambda_dssim
        self.background = tuple(background)
        self.tight_rect = tight_rect
        self.borrow = borrow  # optional BorderExchange (parallel/border.py)
        self.timer = PhaseTimer(self.device, enabled=False)
        self.task_detail = False
        # debug aids (the reference has ``pipe.debug``: a device sync after every launch plus a dump of the rasteriser
        # inputs when it throws, and ``--detect_anomaly`` for NaN hunting; its trainer never switches the former on)
        self.debug = False            # synchronise and read every task's status word after each phase of a step
        self.detect_anomaly = False   # after the backward: non-finite loss sums or gradients raise, naming the sub-model
        self.dump_dir = "."
        # Overflow guard: OR of the overflow words of this step's forwards, on every rank the OR over all ranks by the
        # time the optimiser runs (the peer transport carries the word with its signals, the torch.distributed transport
        # all-reduces it). A step in which any render ran out of instance capacity composited garbage: the fused Adam
        # kernels see the word and drop the update -- on every rank, without a host synchronisation.
        self._skip = torch.zeros(CNT_WORDS, dtype=torch.int32, device=self.device)
        if hasattr(self.transport, "attach_skip"):
            self.transport.attach_skip(self._skip)
        self.dropped_steps = 0
        # occlusion culling between sub-models in the training forward (render_partials_occluded)
        self.occlusion = os.environ.get("RGS_OCCLUSION", "1") == "1"
        self._occl: dict = {}
        self._copy_stream = None
        self._gt_event = None
        self._gt_ready: dict = {}
        self._tasks: dict = {}
        self._grads: dict = {}
        self._closs: dict = {}
        self._gt: dict = {}

    def _task_phase(self, kind: str, cam: Camera, mid: int):
        """With ``task_detail`` the phase timer also keeps one entry per (camera, sub-model) render:
        ``task.<fwd|bwd>:<camera uid>:<sub-model>`` -- the cost matrix behind the load-balance decisions."""
        if self.task_detail and self.timer.enabled:
            return self.timer.phase(f"task.{kind}:{cam.uid}:{mid}")
        return contextlib.nullcontext()

    # -- pools ----------------------------------------------------------------------------------
    def _task(self, view: int, mid: int) -> RenderTask:
        key = (view, mid)
        if key not in self._tasks:
            self._tasks[key] = RenderTask(self.device)
        self._tasks[key].timer = self.timer if self.timer.enabled else None
        return self._tasks[key]

    def _grad(self, view: int, mid: int, H: int, W: int) -> torch.Tensor:
        key = (view, mid)
        g = self._grads.get(key)
        if g is None or g.shape[:2] != (H, W):
            g = torch.zeros(H, W, 4, dtype=torch.float32, device=self.device)
            self._grads[key] = g
        return g

    def _loss(self, view: int, H: int, W: int) -> CompositeLoss:
        cl = self._closs.get(view)
        if cl is None or (cl.H, cl.W) != (H, W):
            cl = CompositeLoss(self.device, H, W)
            self._closs[view] = cl
        # with occlusion culling the backward also stops behind pixels that nearer sub-models finished (the partials of
        # the render tasks carry the mark); without it every partial gets its exact, if tiny, gradient as in the reference
        cl.marked = bool(self.occlusion) and len(self.model2rank) > 1
        return cl

    def _prefetch_gt(self, plans, cams):
        """Start the host -> device copies of this step's ground-truth rows on a copy stream of their own, so that they
        run under the rendering kernels; ``_gt_rows`` then only makes the compute stream wait for them."""
        if self.device.type != "cuda":
            return
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(self.device)
        cur = torch.cuda.current_stream(self.device)
        self._copy_stream.wait_stream(cur)  # the previous step's loss kernels have read the buffers
        with torch.cuda.stream(self._copy_stream):
            for p, cam in zip(plans, cams):
                b = p.bands[self.rank]
                if b[1] > b[0]:
                    self._gt_rows(p.view, cam, (max(0, b[0] - 5), min(p.H, b[1] + 5)))
                    self._gt_ready[p.view] = (cam.uid, b)
        self._gt_event = torch.cuda.Event()
        self._gt_event.record(self._copy_stream)

    def _gt_rows(self, view: int, cam: Camera, rows: tuple[int, int]) -> torch.Tensor:
        """Device (3,H,W) buffer with the ground truth uploaded on ``rows`` only (pinned host -> device)."""
        H, W = cam.height, cam.width
        buf = self._gt.get(view)
        if buf is None or buf.shape != (3, H, W):
            buf = torch.zeros(3, H, W, dtype=torch.float32, device=self.device)
            self._gt[view] = buf
        if self._gt_event is not None and self._gt_ready.get(view) is not None and \
                torch.cuda.current_stream(self.device) != self._copy_stream:
            # uploaded ahead by _prefetch_gt: wait for the copy stream instead of copying again
            self._gt_ready.pop(view)
            torch.cuda.current_stream(self.device).wait_event(self._gt_event)
            return buf
        if cam.image is not None and rows[1] > rows[0]:
            src = cam.image
            if src.device == buf.device:
                buf[:, rows[0]:rows[1]].copy_(src[:, rows[0]:rows[1]])
            else:
                # one copy per colour plane: a band of a plane is contiguous on both sides, so the pinned source goes
                # through the copy engine asynchronously (a strided band would be staged through pageable memory)
                for c in range(3):
                    buf[c, rows[0]:rows[1]].copy_(src[c, rows[0]:rows[1]], non_blocking=True)
        return buf

    # -- segments -------------------------------------------------------------------------------
    def _segments(self, mid: int, with_grads: bool) -> list[Segment]:
        segs = [self.stores[mid].segment(with_grads=with_grads)]
        if self.borrow is not None:
            b = self.borrow.segment(mid, with_grads=with_grads)
            if b is not None and b.count:
                segs.append(b)
        return segs

    def plan(self, cams: list[Camera], relations) -> list[ViewPlan]:
        """``relations[i][m]`` = front-to-back position of sub-model m for camera i, or -1 (invisible)."""
        plans = []
        for i, cam in enumerate(cams):
            rel = [int(v) for v in relations[i]]
            vis = sorted((r, m) for m, r in enumerate(rel) if r >= 0)
            models = [m for _, m in vis]
            plans.append(ViewPlan(i, cam.height, cam.width, models, [self.model2rank[m] for m in models],
                                  band_rows(cam.height, self.world)))
        return plans

    # -- forward --------------------------------------------------------------------------------
    def render_partials(self, cams: list[Camera], plans: list[ViewPlan], sh_degree: int, want_depth: bool = False,
                        check: bool = False) -> dict:
        local_out: dict[int, dict[int, torch.Tensor]] = {}
        for p, cam in zip(plans, cams):
            local_out[p.view] = {}
            for m, r in zip(p.models, p.ranks):
                if r != self.rank:
                    continue
                st = self.stores[m]
                c = make_camera(cam, sh_degree, st.box_lo, st.box_hi, raw_params=True, tight_rect=self.tight_rect)
                task = self._task(p.view, m)
                push = self.transport.push_plan(p, m) if hasattr(self.transport, "push_plan") else None
                with self._task_phase("fwd", cam, m):
                    local_out[p.view][m] = task.forward(c, self._segments(m, False), want_depth=want_depth, check=check,
                                                        push=push)
        return local_out

    def render_partials_occluded(self, cams: list[Camera], plans: list[ViewPlan], sh_degree: int) -> dict:
        """Training forward with occlusion culling between sub-models (``self.occlusion``).

        A sub-model cannot see by itself that nearer sub-models have already finished a tile (every pixel below the
        transmittance threshold), so it bins and blends splats that cannot change the composite by more than that
        threshold. Here every render publishes one byte per tile, "finished", and renders behind it skip those tiles:

        1. every local (view, sub-model), front to back: projection + near slab, skipping the tiles that nearer local
           sub-models finished in their near slabs;
        2. the maps of all sub-models are exchanged (a few KB per map; peer stores + the flag barrier, or one
           all-reduce with the torch.distributed transport);
        3. every local (view, sub-model), front to back: far slab on the tiles that neither its own near slab nor any
           nearer sub-model has finished -- remote ones as of their near slab, local ones as of their whole render.

        Nothing depends on a chain over ranks: one exchange per step. The composite differs from the one without
        culling by at most the transmittance threshold times a colour, like a single render that stops at that threshold."""
        tasks, maps = {}, {}
        for p, cam in zip(plans, cams):
            chain = None
            for m, r in zip(p.models, p.ranks):
                if r != self.rank:
                    continue
                st = self.stores[m]
                c = make_camera(cam, sh_degree, st.box_lo, st.box_hi, raw_params=True, tight_rect=self.tight_rect)
                task = self._task(p.view, m)
                with self._task_phase("fwd", cam, m):
                    task.forward_near(c, self._segments(m, False), occl=chain)
                tasks[(p.view, m)] = task
                maps[(p.view, m)] = task.tile_done
                chain = task.tile_done  # own finished tiles | what was hidden for it: all that is hidden for the next one
        with self.timer.phase("exchange_maps"):
            maps = self.transport.exchange_done_maps(plans, maps)
        local_out: dict[int, dict[int, torch.Tensor]] = {}
        for p, cam in zip(plans, cams):
            local_out[p.view] = {}
            for k, (m, r) in enumerate(zip(p.models, p.ranks)):
                if r != self.rank:
                    continue
                task = tasks[(p.view, m)]
                nearer = [maps[(p.view, j)] for j in p.models[:k]]
                occl = None
                if nearer:
                    occl = self._occl_buf(p.view, m, nearer[0].numel())
                    native.call("tile_maps_or", self.device, native.pointer_array(nearer), len(nearer), occl, occl.numel(), 1,
                                sig="pipiip")
                push = self.transport.push_plan(p, m) if hasattr(self.transport, "push_plan") else None
                with self._task_phase("fwd", cam, m):
                    local_out[p.view][m] = task.forward_far(occl, push=push)
        return local_out

    def _occl_buf(self, view: int, mid: int, n: int) -> torch.Tensor:
        key = (view, mid)
        b = self._occl.get(key)
        if b is None or b.numel() != n:
            b = torch.zeros(n, dtype=torch.uint8, device=self.device)
            self._occl[key] = b
        return b

    def _use_occlusion(self, cams, plans) -> bool:
        if not self.occlusion or len(self.model2rank) < 2:
            return False
        return all(RenderTask.can_split(make_camera(cam, 0, tight_rect=self.tight_rect)) for cam in cams)

    def render(self, cams: list[Camera], relations, sh_degree: int, background=None, want_depth: bool = False):
        """Eval-time render: returns per view the composited (3,H,W) image rows this rank owns
        (``image``, ``rows``) -- with world size 1 that is the whole image.

        ``want_depth`` adds the composited depth ``sum_k T_<k D_k`` and ``alpha = 1 - T_total`` on the same rows
        (``result_aggregator.py:244-259`` of the reference). The depth partials travel as a second 4-channel
        image (D_k, 0, 0, T_k) through the same ordered "over": its first channel composites to exactly that sum."""
        bg = self.background if background is None else background
        plans = self.plan(cams, relations)
        self._prepare_transport(plans)
        if self.borrow is not None:
            self.borrow.refresh(self.stores, need_grads=False)
        if self._use_occlusion(cams, plans) and not want_depth:
            # the culled forward runs unchecked: all ranks look at the step's overflow word together (it travels with the
            # exchange) and repeat the render with grown buffers when any render ran out of instance capacity
            for attempt in range(8):
                local_out = self.render_partials_occluded(cams, plans, sh_degree)
                self._collect_overflow(plans)
                slots = self.transport.exchange_partials(plans, local_out)
                overflow = bool(int(self._skip[CNT_OVERFLOW].item()))
                self.poll()
                if not overflow:
                    break
                self.transport.barrier()
            else:
                raise RuntimeError("the instance buffers still overflow after 8 attempts to grow them")
        else:
            local_out = self.render_partials(cams, plans, sh_degree, want_depth=want_depth, check=True)
            slots = self.transport.exchange_partials(plans, local_out)
        out = []
        for p in plans:
            cl = self._loss(p.view, p.H, p.W)
            b = p.bands[self.rank]
            if b[1] > b[0]:  # five more rows on each side so that SSIM windows of the band are complete
                cl.composite(slots[p.view], bg, max(0, b[0] - 5), min(p.H, b[1] + 5))
            out.append(dict(image=cl.image, trans=cl.trans, rows=b, partials=local_out[p.view], plan=p))
        self.transport.barrier()  # slots may be overwritten by the next render only after everyone composited
        if want_depth:
            dparts = {}
            for p in plans:
                dparts[p.view] = {}
                for m, part in local_out[p.view].items():
                    d4 = torch.zeros_like(part)
                    d4[..., 0] = self._tasks[(p.view, m)].depth
                    d4[..., 3] = part[..., 3]
                    dparts[p.view][m] = d4
            move = getattr(self.transport, "exchange_images", self.transport.exchange_partials)
            dslots = move(plans, dparts)
            for p, o in zip(plans, out):
                b = p.bands[self.rank]
                dimg = torch.zeros(3, p.H, p.W, dtype=torch.float32, device=self.device)
                dtr = torch.ones(p.H, p.W, dtype=torch.float32, device=self.device)
                if b[1] > b[0]:
                    self._loss(p.view, p.H, p.W).composite(dslots[p.view], (0.0, 0.0, 0.0), b[0], b[1], image=dimg, trans=dtr)
                o["depth"], o["alpha"] = dimg[0], 1.0 - dtr
            self.transport.barrier()
        return out

    def _prepare_transport(self, plans):
        if hasattr(self.transport, "prepare") and plans:
            self.transport.prepare(plans, len(self.model2rank), self.model2rank)

    # -- training step --------------------------------------------------------------------------
    def train_step(self, cams: list[Camera], relations, sh_degree: int, lrs, optimizer_step: bool = True,
                   background=None) -> StepResult:
        bg = self.background if background is None else background
        T = self.timer.phase
        plans = self.plan(cams, relations)
        self._prepare_transport(plans)
        self._prefetch_gt(plans, cams)
        if self.borrow is not None:
            if hasattr(self.borrow, "timer"):
                self.borrow.timer = self.timer
            with T("border_exchange"):
                self.borrow.refresh(self.stores, need_grads=True)
        with T("render_forward"):
            if self._use_occlusion(cams, plans):
                local_out = self.render_partials_occluded(cams, plans, sh_degree)
            else:
                local_out = self.render_partials(cams, plans, sh_degree)
            self._collect_overflow(plans)
        with T("exchange_partials"):
            slots = self.transport.exchange_partials(plans, local_out)
        if hasattr(self.transport, "local_grad_images"):
            local_grad = self.transport.local_grad_images(plans)
        else:
            local_grad = {p.view: {m: self._grad(p.view, m, p.H, p.W) for m, r in zip(p.models, p.ranks)
                                   if r == self.rank} for p in plans}
        gslots = self.transport.grad_slots(plans, local_grad)
        sums = []
        with T("composite_loss"):
            for p, cam in zip(plans, cams):
                cl = self._loss(p.view, p.H, p.W)
                b = p.bands[self.rank]
                if b[1] <= b[0]:
                    sums.append(torch.zeros(3, dtype=torch.float64, device=self.device))
                    continue
                gt = self._gt_rows(p.view, cam, (max(0, b[0] - 5), min(p.H, b[1] + 5)))
                sums.append(cl.fused_loss_backward(slots[p.view], gslots[p.view], gt, bg, self.lambda_dssim, b[0], b[1]).clone())
        if self.debug:
            self._debug_check("forward+loss", cams)
        with T("return_grads"):
            self.transport.return_grads(plans, gslots, local_grad)
        with T("render_backward"):
            for p, cam in zip(plans, cams):
                for m, r in zip(p.models, p.ranks):
                    if r == self.rank:
                        with self._task_phase("bwd", cam, m):
                            self._task(p.view, m).backward(local_grad[p.view][m], self._segments(m, True))
        if self.debug:
            self._debug_check("backward", cams)
        if self.detect_anomaly:
            self._anomaly_check(sums)
        if self.borrow is not None:
            with T("border_return"):
                self.borrow.return_grads(self.stores)
        if optimizer_step:
            self.optimizer_step(lrs, plans)
        return StepResult(sums=sums, plans=plans)

    # -- debug aids -------------------------------------------------------------------------------
    def _debug_check(self, phase: str, cams):
        """Synchronise, read the status words of all render tasks; on an error write the inputs of the step to
        ``snapshot_<phase>.dump`` (cameras and parameters of the local sub-models) and re-raise."""
        try:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            for task in self._tasks.values():
                if task.cam is not None:
                    task._record_counters()
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            for task in self._tasks.values():
                if task.cam is not None:
                    task.poll()
            if hasattr(self.transport, "check"):
                self.transport.check()
        except Exception:
            import os
            path = os.path.join(self.dump_dir, f"snapshot_{phase.replace('+', '_')}.dump")
            torch.save({"phase": phase, "cameras": [c.pack() for c in cams],
                        "models": {m: st.records().cpu() for m, st in self.stores.items()}}, path)
            raise

    def _anomaly_check(self, sums):
        for i, s in enumerate(sums):
            if not bool(torch.isfinite(s).all()):
                raise FloatingPointError(f"non-finite loss sums for view {i} of the batch: {s.tolist()}")
        for m, st in self.stores.items():
            g = st.views("grads")
            for name, t in g.items():
                if t.numel() and not bool(torch.isfinite(t).all()):
                    bad = int((~torch.isfinite(t)).any(dim=1).nonzero()[0])
                    raise FloatingPointError(f"non-finite gradient in sub-model {m}, group '{name}', first at Gaussian {bad}")

    def _collect_overflow(self, plans):
        """Fold the overflow words of this step's forwards into the step's skip word (see ``__init__``)."""
        cnts = [self._tasks[(p.view, m)].counters for p in plans for m, r in zip(p.models, p.ranks) if r == self.rank]
        flags = self._skip[CNT_OVERFLOW:CNT_OVERFLOW + 2]  # overflow and status word; the counts are not flags
        if cnts:
            torch.amax(torch.stack([c[CNT_OVERFLOW:CNT_OVERFLOW + 2] for c in cnts]), dim=0, out=flags)
        else:
            flags.zero_()
        if hasattr(self.transport, "reduce_skip"):
            self.transport.reduce_skip(self._skip)

    def optimizer_step(self, lrs, plans=None):
        with self.timer.phase("adam"):
            for m, st in self.stores.items():
                st.adam_step(lrs, skip=self._skip)
        self._record_step_status()

    def _record_step_status(self):
        """Queue copies of the skip word and of the transport's wait status to the host (read by ``poll_async``)."""
        if self.device.type == "cuda":
            if not hasattr(self, "_host_skip"):
                self._host_skip = torch.zeros(CNT_WORDS, dtype=torch.int32).pin_memory()
            self._host_skip.copy_(self._skip, non_blocking=True)
            self._skip_event = torch.cuda.Event()
            self._skip_event.record(torch.cuda.current_stream(self.device))
            if hasattr(self.transport, "record_status"):
                self.transport.record_status()

    def poll_async(self) -> dict | None:
        """Look at the counters of the last step whose copies have reached the host, without waiting for the device:
        grows instance buffers that overflowed or came close (applied by the next forward), raises when a bounded wait of
        the transport gave up, and tells whether that step's optimiser update was dropped. ``None`` while the copies
        are still in flight (the step is then looked at by a later call)."""
        if self.device.type != "cuda":
            info = self.poll()
            info["dropped"] = bool(self._skip[CNT_OVERFLOW])
            self.dropped_steps += int(info["dropped"])
            return info
        ev = getattr(self, "_skip_event", None)
        if ev is None or not ev.query():
            return None
        self._skip_event = None
        info = self.poll()
        info["dropped"] = bool(self._host_skip[CNT_OVERFLOW])
        self.dropped_steps += int(info["dropped"])
        if hasattr(self.transport, "check"):
            self.transport.check(block=False)
        return info

    def poll(self) -> dict:
        """After a host synchronisation: read the counters of all tasks (grows buffers when needed)."""
        info = dict(overflow=False, n_vis=0, n_inst=0)
        for task in self._tasks.values():
            if task.cam is None:
                continue
            c = task.poll()
            info["overflow"] |= c["overflow"]
            info["n_vis"] += c["n_vis"]
            info["n_inst"] += c["n_inst"]
        return info
