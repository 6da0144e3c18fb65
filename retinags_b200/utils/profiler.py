"""Per-phase timing and tracing.

``PhaseTimer`` brackets the phases of a step with CUDA events on the launching stream (no host
synchronisation until the numbers are read) and NVTX ranges, so a step can be read in a profiler timeline or
reduced to a per-phase table (maximum over ranks for multi-GPU numbers), or written as a Chrome trace
(``chrome://tracing`` / Perfetto JSON: one complete event per phase on the device's own time base).  On CPU ranks it
falls back to ``time.perf_counter``.  The reference only has a whole-iteration CUDA-event timer
(``trainer4tree_partition.py:590,613,641-643``) and an unused ``NaiveTimer`` (``utils/workload_utils.py:61-81``).
"""
from __future__ import annotations

import contextlib
import json
import time
from collections import defaultdict

import torch


class PhaseTimer:
    def __init__(self, device, enabled: bool = False, nvtx: bool = True):
        self.device = torch.device(device)
        self.enabled = enabled
        self.cuda = self.device.type == "cuda"
        self.nvtx = nvtx and self.cuda
        self._pending: list[tuple[str, object, object]] = []
        self.totals: dict[str, float] = defaultdict(float)
        self.host_totals: dict[str, float] = defaultdict(float)  # wall clock of the host inside the phase (ms)
        self.counts: dict[str, int] = defaultdict(int)
        self.trace = False              # keep every phase instance for export_chrome_trace
        self.events: list[tuple[str, float, float]] = []  # (name, start ms, duration ms) relative to the first phase
        self._origin = None

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        h0 = time.perf_counter()
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(torch.cuda.current_stream(self.device))
            if self.trace and self._origin is None:
                self._origin = a
        else:
            a, b = time.perf_counter(), None
            if self.trace and self._origin is None:
                self._origin = a
        try:
            yield
        finally:
            self.host_totals[name] += (time.perf_counter() - h0) * 1e3
            if self.cuda:
                b.record(torch.cuda.current_stream(self.device))
                self._pending.append((name, a, b))
            else:
                now = time.perf_counter()
                self.totals[name] += (now - a) * 1e3
                self.counts[name] += 1
                if self.trace:
                    self.events.append((name, (a - self._origin) * 1e3, (now - a) * 1e3))
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    def collect(self) -> dict[str, float]:
        """Fold the pending event pairs into ``totals`` (synchronises the device once)."""
        if self.cuda and self._pending:
            torch.cuda.synchronize(self.device)
            for name, a, b in self._pending:
                dur = a.elapsed_time(b)
                self.totals[name] += dur
                self.counts[name] += 1
                if self.trace and self._origin is not None:
                    self.events.append((name, self._origin.elapsed_time(a), dur))
            self._pending.clear()
        return dict(self.totals)

    def reset(self):
        self._pending.clear()
        self.totals.clear()
        self.host_totals.clear()
        self.counts.clear()
        self.events.clear()
        self._origin = None

    def export_chrome_trace(self, path: str, rank: int = 0):
        """Write the recorded phase instances (``trace = True``) as complete events; nested phases nest in the viewer."""
        self.collect()
        ev = [{"name": n, "ph": "X", "ts": start * 1e3, "dur": dur * 1e3, "pid": rank, "tid": 0, "cat": "phase"}
              for n, start, dur in sorted(self.events, key=lambda e: e[1])]
        ev.insert(0, {"name": "process_name", "ph": "M", "pid": rank, "args": {"name": f"rank {rank} ({self.device})"}})
        with open(path, "w") as f:
            json.dump({"traceEvents": ev, "displayTimeUnit": "ms"}, f)

    def table(self, steps: int = 1, group=None) -> dict[str, float]:
        """ms per step and phase; with a process group the maximum over ranks."""
        tot = self.collect()
        names = sorted(tot)
        vals = torch.tensor([tot[n] / max(steps, 1) for n in names], dtype=torch.float64,
                            device=self.device if self.cuda else "cpu")
        if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
            torch.distributed.all_reduce(vals, op=torch.distributed.ReduceOp.MAX, group=group)
        return {n: float(v) for n, v in zip(names, vals.tolist())}
