"""Movement of partial images to their owners and of their gradients back.

Ownership is by *row band*: every view is cut into ``world`` horizontal bands whose borders sit on
multiples of the 16-row tile height, and rank ``r`` owns band ``r`` of every view of the batch.
An owner needs the partial images on its band plus one tile row on each side (the D-SSIM window
reaches 5 rows, its gradient 10), composites them in depth order, evaluates the loss on its own
rows and returns ``dL/d(partial)`` for those rows to each contributing rank.  Ingress is therefore
spread evenly over the GPUs instead of converging on one "main rank" per view as in the reference
(``parallel_utils/basic_parallel_trainer/task_utils.py:57-93``,
``trainer4tree_partition.py:390-415,466-516``), whose (5,H,W) partials all travel to rank
``i % world``.

Transports:

* ``LocalTransport``      world size 1: slots alias the render outputs, nothing moves.
* ``TorchDistTransport``  ``batch_isend_irecv`` of row slices (NCCL on GPUs, gloo on CPU ranks).  It
  reproduces the reference's communication pattern (``communicate_utils/core.py:37-65``) and is the
  in-repo baseline and the CPU test vehicle.
* ``PeerTransport`` (``parallel/peer.py``) the fused path: the blend kernel's epilogue stores tiles
  straight into the owner's slot through peer-mapped memory, the compositing backward stores
  gradient rows straight into the source's gradient image.
"""
from __future__ import annotations

from dataclasses import dataclass

import os

import torch
import torch.distributed as dist

TILE = 16
HALO_ROWS = TILE


def band_rows(H: int, world: int) -> list[tuple[int, int]]:
    """Row range [r0,r1) of every rank's band; borders are multiples of the tile height."""
    tiles = (H + TILE - 1) // TILE
    base, extra = divmod(tiles, world)
    out, t = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((min(t * TILE, H), min((t + n) * TILE, H)))
        t += n
    return out


def extended(band: tuple[int, int], H: int) -> tuple[int, int]:
    """Rows an owner needs of every partial: its band plus one tile row on each side."""
    if band[1] <= band[0]:
        return band
    return max(0, band[0] - HALO_ROWS), min(H, band[1] + HALO_ROWS)


@dataclass
class ViewPlan:
    """Who contributes what to one view of the batch."""

    view: int                 # index inside the batch
    H: int
    W: int
    models: list[int]         # visible sub-models in front-to-back order
    ranks: list[int]          # rank hosting each of them
    bands: list[tuple[int, int]]


class LocalTransport:
    world = 1
    rank = 0

    def __init__(self, device):
        self.device = torch.device(device)

    def partial_slots(self, plan: ViewPlan, local_out: dict[int, torch.Tensor]) -> list[torch.Tensor]:
        return [local_out[m] for m in plan.models]

    def exchange_partials(self, plans, local_out):
        return {p.view: self.partial_slots(p, local_out[p.view]) for p in plans}

    def grad_slots(self, plans, local_grad):
        return {p.view: [local_grad[p.view][m] for m in p.models] for p in plans}

    def return_grads(self, plans, slots, local_grad):
        return None

    def exchange_done_maps(self, plans, local_maps):
        """{(view, model): uint8 map of finished tiles} of every visible sub-model; all are local here."""
        return dict(local_maps)

    def barrier(self):
        return None


class TorchDistTransport:
    """Row-slice send/recv of partials and gradients with ``torch.distributed`` point-to-point ops."""

    def __init__(self, device, group=None, version: str | None = None):
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self._pool: dict = {}
        # how a batch of point-to-point operations is issued (the reference's communicate_utils/core.py:37-233):
        #   "0"            one batch_isend_irecv, wait for all (its default)
        #   "0+profiling"  the same inside a profiler range
        #   "1"            blocking send/recv, peer by peer, the lower rank sends first (cannot deadlock)
        #   "2"            all irecv posted first, then all isend, then wait
        self.version = version if version is not None else os.environ.get("RGS_COMM_VERSION", "0")
        if self.version not in ("0", "0+profiling", "1", "2"):
            raise ValueError(f"unknown communication version {self.version!r}")

    def _buf(self, key, shape):
        t = self._pool.get(key)
        if t is None or tuple(t.shape) != tuple(shape):
            t = torch.zeros(*shape, dtype=torch.float32, device=self.device)
            self._pool[key] = t
        return t

    def _run(self, ops):
        if not ops:
            return
        if self.version == "0":
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        elif self.version == "0+profiling":
            with torch.profiler.record_function("batched_send_recv"):
                for req in dist.batch_isend_irecv(ops):
                    req.wait()
        elif self.version == "1":
            # both ends walk their common operations in the order in which they were queued; towards a higher rank
            # this rank sends first, towards a lower one it receives first
            peers = sorted({op.peer for op in ops})
            for peer in peers:
                mine = [op for op in ops if op.peer == peer]
                sends = [op for op in mine if op.op is dist.isend]
                recvs = [op for op in mine if op.op is dist.irecv]
                first, second = (sends, recvs) if self.rank < peer else (recvs, sends)
                for op in first + second:
                    (dist.send if op.op is dist.isend else dist.recv)(op.tensor, peer, group=self.group)
        else:
            reqs = [dist.irecv(op.tensor, op.peer, group=self.group) for op in ops if op.op is dist.irecv]
            reqs += [dist.isend(op.tensor, op.peer, group=self.group) for op in ops if op.op is dist.isend]
            for req in reqs:
                req.wait()

    def exchange_partials(self, plans: list[ViewPlan], local_out: dict[int, dict[int, torch.Tensor]]):
        """Returns {view: [slot per visible model]}; a slot is a *full-height virtual* (H,W,4) view of
        which only the owner's extended rows are backed by valid data."""
        ops, result = [], {}
        for p in plans:
            slots = []
            my_ext = extended(p.bands[self.rank], p.H)
            for m, r in zip(p.models, p.ranks):
                if r == self.rank:
                    part = local_out[p.view][m]
                    slots.append(part)
                    for o in range(self.world):
                        e = extended(p.bands[o], p.H)
                        if o != self.rank and e[1] > e[0]:
                            ops.append(dist.P2POp(dist.isend, part[e[0]:e[1]], o, self.group))
                else:
                    if my_ext[1] > my_ext[0]:
                        full = self._buf(("p", p.view, m), (p.H, p.W, 4))
                        ops.append(dist.P2POp(dist.irecv, full[my_ext[0]:my_ext[1]], r, self.group))
                        slots.append(full)
                    else:
                        slots.append(self._buf(("p", p.view, m), (p.H, p.W, 4)))
            result[p.view] = slots
        self._run(ops)
        return result

    def grad_slots(self, plans, local_grad):
        """Where the owner writes dL/d(partial): the local gradient image for local models, a staging
        buffer for remote ones."""
        out = {}
        for p in plans:
            out[p.view] = [local_grad[p.view][m] if r == self.rank else self._buf(("g", p.view, m), (p.H, p.W, 4))
                           for m, r in zip(p.models, p.ranks)]
        return out

    def return_grads(self, plans, slots, local_grad):
        ops = []
        for p in plans:
            b = p.bands[self.rank]
            for k, (m, r) in enumerate(zip(p.models, p.ranks)):
                if r == self.rank:
                    for o in range(self.world):
                        ob = p.bands[o]
                        if o != self.rank and ob[1] > ob[0]:
                            ops.append(dist.P2POp(dist.irecv, local_grad[p.view][m][ob[0]:ob[1]], o, self.group))
                elif b[1] > b[0]:
                    ops.append(dist.P2POp(dist.isend, slots[p.view][k][b[0]:b[1]], r, self.group))
        self._run(ops)

    def exchange_done_maps(self, plans, local_maps):
        """Every rank receives the finished-tile maps (uint8 per tile) of all visible sub-models: one all-reduce (MAX)
        of a buffer in which each rank has filled in the maps of its own sub-models."""
        out, bufs = dict(local_maps), []
        for p in plans:
            tiles = ((p.H + TILE - 1) // TILE) * ((p.W + TILE - 1) // TILE)
            buf = torch.zeros(len(p.models), tiles, dtype=torch.uint8, device=self.device)
            for k, (m, r) in enumerate(zip(p.models, p.ranks)):
                if r == self.rank:
                    buf[k].copy_(local_maps[(p.view, m)])
            bufs.append(buf)
        if bufs:
            flat = torch.cat([b.reshape(-1) for b in bufs])
            dist.all_reduce(flat, op=dist.ReduceOp.MAX, group=self.group)
            off = 0
            for p, b in zip(plans, bufs):
                got = flat[off:off + b.numel()].view_as(b)
                off += b.numel()
                for k, (m, r) in enumerate(zip(p.models, p.ranks)):
                    if r != self.rank:
                        out[(p.view, m)] = got[k]
        return out

    def reduce_skip(self, skip: torch.Tensor):
        """Every rank leaves with the maximum over ranks of the step's overflow word (queued on the stream)."""
        dist.all_reduce(skip, op=dist.ReduceOp.MAX, group=self.group)

    def barrier(self):
        dist.barrier(self.group)
