"""Parameter store of one sub-model.

All optimisable state of a sub-model lives in four flat fp32 buffers of identical layout
(parameters, gradients, Adam first and second moments).  A buffer holds five column groups of
``cap`` rows each -- xyz(3) | sh(48, coefficient-major) | log-scale(3) | rotation(4, wxyz) |
opacity-logit(1) -- so a render kernel streams exactly the columns it needs (culled Gaussians cost
12 bytes), and one fused Adam launch covers all 59 columns.  The reference keeps seven separate
``nn.Parameter`` tensors per sub-model with a per-tensor ``torch.optim.Adam``
(``scene/gaussian_nn_module.py:296-452``) and re-creates the optimiser state with ``cat``/mask
surgery on every densification (``:589-664``); here the same surgery is an index gather on the
four buffers.

Record layouts (row-major, for files and for migration between sub-models) follow the reference:
59 floats ``xyz f_dc f_rest(15x3) scaling rotation opacity`` (``gaussian_nn_module.py:839-847``)
and 177 floats ``[params, exp_avg, exp_avg_sq]`` (``:849-870``).
"""
from __future__ import annotations

import math
import os

import torch

from ..ops import native
from ..ops.rasterize import Segment

WIDTHS = (3, 48, 3, 4, 1)
NAMES = ("xyz", "sh", "scale", "rot", "opacity")
RECORD = 59


def _round_cap(n: int) -> int:
    return max(4, (int(n) + 3) // 4 * 4)


_ADAM_ROWS_OK: dict[str, bool] = {}


def adam_rows_agrees(device) -> bool:
    """One-off check per device: the row-block Adam kernel and the per-unit kernel, run on the same small store with
    sparse marks, dense marks and a ragged tail, must leave every buffer identical bit for bit. The result is cached;
    a disagreement (or any error) selects the per-unit kernel and is reported once."""
    key = str(device)
    if key in _ADAM_ROWS_OK:
        return _ADAM_ROWS_OK[key]
    _ADAM_ROWS_OK[key] = False  # also guards against re-entry while the check runs
    try:
        gen = torch.Generator().manual_seed(1234)
        n = 1001
        stores = []
        for variant in ("units", "rows"):
            st = GaussianStore(n, device)
            st.adam_variant = variant
            st.count = n
            stores.append(st)
        init = torch.randn(stores[0].params.shape, generator=gen)
        for st in stores:
            st.params.copy_(init)
        lrs = (1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2)
        for step in range(4):
            grads = torch.randn(stores[0].grads.shape, generator=gen) * 1e-3
            rows = torch.arange(0, n, 7 if step < 2 else 1)
            for st in stores:
                st.grads.copy_(grads)
                keep = torch.zeros(st.cap, dtype=torch.bool, device=st.device)
                keep[rows.to(st.device)] = True
                for view in dict(GaussianStore._views(st.grads, st.cap, st.cap)).values():
                    view[~keep] = 0
                st.mark_touched(rows.to(st.device))
                st.adam_step(lrs)
        for st in stores:  # and one dense step without marks
            st.grads.copy_(grads)
            st.adam_step(lrs, zero_grad=False)
        a, b = stores
        diff = first_store_difference(a, b)
        _ADAM_ROWS_OK[key] = diff is None
        if diff is not None:
            import warnings
            warnings.warn("the row-block Adam kernel disagrees with the per-unit kernel on this device; using the latter "
                          f"(first difference: {diff})")
    except Exception as exc:  # keep training on the validated kernel
        import warnings
        warnings.warn(f"the check of the row-block Adam kernel failed ({exc!r}); using the per-unit kernel")
    return _ADAM_ROWS_OK[key]


def first_store_difference(a: "GaussianStore", b: "GaussianStore") -> str | None:
    """Where two stores of equal shape first differ bit for bit: buffer, column group, row, column and the two bit
    patterns; ``None`` when parameters, gradients, both moments and the ``active`` marks are identical."""
    for which in ("params", "grads", "exp_avg", "exp_avg_sq"):
        va, vb = a.views(which), b.views(which)
        for name in NAMES:
            xa, xb = va[name].contiguous().view(torch.int32), vb[name].contiguous().view(torch.int32)
            ne = (xa != xb)
            if bool(ne.any()):
                row, col = [int(x) for x in ne.nonzero()[0]]
                return (f"{which}.{name} row {row} column {col}: {int(xa[row, col]) & 0xFFFFFFFF:#010x} vs "
                        f"{int(xb[row, col]) & 0xFFFFFFFF:#010x} ({int(ne.sum())} of {ne.numel()} words differ)")
    ne = a.active[:a.count] != b.active[:b.count]
    if bool(ne.any()):
        row = int(ne.nonzero()[0])
        return f"active row {row}: {int(a.active[row])} vs {int(b.active[row])}"
    return None


class GaussianStore:
    def __init__(self, capacity: int, device, sh_degree: int = 3, box_lo=None, box_hi=None, model_id: int = 0):
        self.device = torch.device(device)
        self.max_sh_degree = sh_degree
        self.active_sh_degree = 0
        self.model_id = model_id
        self.box_lo = [-math.inf] * 3 if box_lo is None else [float(v) for v in box_lo]
        self.box_hi = [math.inf] * 3 if box_hi is None else [float(v) for v in box_hi]
        self.count = 0
        self.cap = 0
        self.step = 0
        self.params = self.grads = self.exp_avg = self.exp_avg_sq = None
        self.grad_accum = self.denom = self.max_radii = None
        # "units": one thread per 128-bit unit; "rows": a warp per 32 rows that skips dead rows after one ballot
        # (csrc/rgs_model.cu: rgs_adam_rows_kernel, much cheaper when few rows are live); "auto": "rows" on CUDA devices
        # on which a one-off comparison of the two kernels agreed bit for bit, "units" otherwise
        self.adam_variant = os.environ.get("RGS_ADAM", "auto")
        self._live_list = self._live_count = None
        self.touched = None  # uint8 per row: a gradient was written this step (rows with 0 hold zero gradients)
        self.active = None   # uint8 per row: the Adam moments may be non-zero (rows with 0 hold zero moments)
        self._alloc(_round_cap(capacity))

    # -- storage --------------------------------------------------------------------------------
    def _alloc(self, cap: int):
        dev = self.device
        old = (self.params, self.grads, self.exp_avg, self.exp_avg_sq, self.cap, self.count)
        old_stats = (self.grad_accum, self.denom, self.max_radii, self.active)
        self.cap = cap
        self.params = torch.zeros(RECORD * cap, dtype=torch.float32, device=dev)
        self.grads = torch.zeros(RECORD * cap, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(RECORD * cap, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(RECORD * cap, dtype=torch.float32, device=dev)
        self.grad_accum = torch.zeros(cap, dtype=torch.float32, device=dev)
        self.denom = torch.zeros(cap, dtype=torch.float32, device=dev)
        self.max_radii = torch.zeros(cap, dtype=torch.float32, device=dev)
        # gradients do not survive a reallocation: the invariant "untouched rows are zero" restarts
        self.touched = torch.zeros(cap, dtype=torch.uint8, device=dev)
        self.active = torch.zeros(cap, dtype=torch.uint8, device=dev)
        if old[0] is not None and old[5] > 0:
            n, ocap = old[5], old[4]
            for new_buf, old_buf in zip((self.params, None, self.exp_avg, self.exp_avg_sq), old[:4]):
                if new_buf is None:
                    continue
                for (_, nv), (_, ov) in zip(self._views(new_buf, cap, n), self._views(old_buf, ocap, n)):
                    nv.copy_(ov)
            for nb, ob in zip((self.grad_accum, self.denom, self.max_radii, self.active), old_stats):
                nb[:n].copy_(ob[:n])

    @staticmethod
    def _views(buf: torch.Tensor, cap: int, count: int):
        off = 0
        for name, w in zip(NAMES, WIDTHS):
            yield name, buf[off:off + cap * w].view(cap, w)[:count]
            off += cap * w

    def views(self, which: str = "params") -> dict:
        return dict(self._views(getattr(self, which), self.cap, self.count))

    def reserve(self, n: int):
        if n > self.cap:
            self._alloc(_round_cap(max(n, int(self.cap * 1.5))))

    # -- content --------------------------------------------------------------------------------
    def set_params(self, g: dict):
        n = int(g["xyz"].shape[0])
        self.reserve(n)
        self.count = n
        for name, v in self.views("params").items():
            v.copy_(g[name].reshape(n, -1).to(self.device))
        for which in ("grads", "exp_avg", "exp_avg_sq"):
            getattr(self, which).zero_()
        self.touched.zero_()
        self.active.zero_()
        self.reset_stats()

    def reset_stats(self):
        self.grad_accum.zero_()
        self.denom.zero_()
        self.max_radii.zero_()

    def __len__(self):
        return self.count

    @property
    def xyz(self):
        return self.views()["xyz"]

    def segment(self, with_grads: bool = True, with_stats: bool = True) -> Segment:
        p = self.views("params")
        seg = Segment(p["xyz"], p["sh"], p["scale"], p["rot"], p["opacity"])
        if with_grads:
            g = self.views("grads")
            seg.g_xyz, seg.g_sh, seg.g_scale, seg.g_rot, seg.g_opacity = g["xyz"], g["sh"], g["scale"], g["rot"], g["opacity"]
            seg.touched = self.touched[:self.count]
            if with_stats:
                seg.stat_grad = self.grad_accum[:self.count]
                seg.stat_denom = self.denom[:self.count]
                seg.stat_maxrad = self.max_radii[:self.count]
        return seg

    # -- records --------------------------------------------------------------------------------
    def records(self, which: str = "params", index: torch.Tensor | None = None) -> torch.Tensor:
        """(n,59) row-major records of the chosen buffer (optionally only rows ``index``)."""
        v = self.views(which)
        cols = [v[name] if index is None else v[name][index] for name in NAMES]
        return torch.cat(cols, dim=1)

    def migration_records(self, index: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """(n,177) = [params, exp_avg, exp_avg_sq] rows, packed by one kernel (``csrc/rgs_surgery.cu``)."""
        n = self.count if index is None else int(index.numel())
        rec = out if out is not None else torch.empty(n, 3 * RECORD, dtype=torch.float32, device=self.device)
        if n:
            idx = None if index is None else index.to(torch.int64).contiguous()
            native.call("records_pack", self.device, self.params, self.exp_avg, self.exp_avg_sq, self.cap, idx, 0, n, rec)
        return rec

    def load_records(self, rec: torch.Tensor, which: str = "params", start: int = 0):
        n = rec.shape[0]
        off = 0
        full = dict(self._views(getattr(self, which), self.cap, self.cap))
        for name, w in zip(NAMES, WIDTHS):
            full[name][start:start + n].copy_(rec[:, off:off + w])
            off += w

    def append_migration(self, rec: torch.Tensor):
        """Append (n,177) migration records (parameters and Adam moments)."""
        n = rec.shape[0]
        if n == 0:
            return
        self.reserve(self.count + n)
        rec = rec.to(self.device, torch.float32).contiguous()
        native.call("records_unpack", self.device, rec, n, self.params, self.exp_avg, self.exp_avg_sq, self.cap, self.count)
        for s in (self.grad_accum, self.denom, self.max_radii):
            s[self.count:self.count + n] = 0
        self.active[self.count:self.count + n] = 1  # the records carry moments
        self.count += n

    # -- surgery --------------------------------------------------------------------------------
    def keep(self, mask_or_index: torch.Tensor):
        """Keep the selected rows (stable order) in all buffers and statistics."""
        idx = mask_or_index.nonzero(as_tuple=True)[0] if mask_or_index.dtype == torch.bool else mask_or_index
        n = int(idx.numel())
        self.zero_grad()  # surgery drops the gradients of the step
        for which in ("params", "exp_avg", "exp_avg_sq"):
            buf = getattr(self, which)
            full = dict(self._views(buf, self.cap, self.cap))
            for name in NAMES:
                full[name][:n] = full[name][idx]
        for s in (self.grad_accum, self.denom, self.max_radii, self.active):
            s[:n] = s[idx]
        self.count = n

    def spatial_sort(self, bits: int = 16) -> torch.Tensor | None:
        """Reorder the rows along a Morton (Z-order) curve through their positions, in all buffers and statistics.

        A camera sees a compact region of space, and the render kernels fetch the rows of the visible Gaussians (236
        bytes each, from five column groups): with rows in the order of a space-filling curve those fetches fall into
        a few contiguous stretches of each group instead of being spread evenly over gigabytes. The reference keeps
        the order of the input file (``scene/gaussian_nn_module.py:134-174``). Call between steps only (it drops the
        gradients of the step like any other surgery); returns the permutation that was applied."""
        n = self.count
        if n < 2:
            return None
        xyz = self.views()["xyz"]
        lo, hi = xyz.min(0).values, xyz.max(0).values
        q = ((xyz - lo) / (hi - lo).clamp_min(1e-12) * ((1 << bits) - 1)).round().clamp_(0, (1 << bits) - 1).to(torch.int64)

        def spread(v):  # bit k of a 21-bit value -> bit 3k
            v = (v | (v << 32)) & 0x1F00000000FFFF
            v = (v | (v << 16)) & 0x1F0000FF0000FF
            v = (v | (v << 8)) & 0x100F00F00F00F00F
            v = (v | (v << 4)) & 0x10C30C30C30C30C3
            v = (v | (v << 2)) & 0x1249249249249249
            return v

        key = spread(q[:, 0]) | (spread(q[:, 1]) << 1) | (spread(q[:, 2]) << 2)
        perm = torch.argsort(key, stable=True)
        del key, q
        self.keep(perm)
        return perm

    def adopt(self, params: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, cap: int, count: int,
              with_moments: int = 0):
        """Take over freshly written buffers of ``cap`` rows (the output of the compaction kernels): gradients and
        statistics restart from zero; the first ``with_moments`` rows carry Adam moments."""
        dev = self.device
        self.params, self.exp_avg, self.exp_avg_sq = params, exp_avg, exp_avg_sq
        self.cap, self.count = cap, count
        self.grads = torch.zeros(RECORD * cap, dtype=torch.float32, device=dev)
        self.grad_accum = torch.zeros(cap, dtype=torch.float32, device=dev)
        self.denom = torch.zeros(cap, dtype=torch.float32, device=dev)
        self.max_radii = torch.zeros(cap, dtype=torch.float32, device=dev)
        self.touched = torch.zeros(cap, dtype=torch.uint8, device=dev)
        self.active = torch.zeros(cap, dtype=torch.uint8, device=dev)
        self.active[:with_moments] = 1

    def append_new(self, g: dict):
        """Append freshly created Gaussians (zero moments, zero statistics)."""
        n = int(g["xyz"].shape[0])
        if n == 0:
            return
        self.reserve(self.count + n)
        full = dict(self._views(self.params, self.cap, self.cap))
        for name in NAMES:
            full[name][self.count:self.count + n] = g[name].reshape(n, -1)
        for which in ("grads", "exp_avg", "exp_avg_sq"):
            fullw = dict(self._views(getattr(self, which), self.cap, self.cap))
            for name in NAMES:
                fullw[name][self.count:self.count + n] = 0
        for s in (self.grad_accum, self.denom, self.max_radii, self.active):
            s[self.count:self.count + n] = 0
        self.count += n

    # -- optimiser ------------------------------------------------------------------------------
    def adam_step(self, lrs, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-15, skip: torch.Tensor | None = None,
                  zero_grad: bool = True):
        """One fused Adam update over all 59 columns; ``lrs`` = (xyz, f_dc, f_rest, scale, rot, opacity)."""
        self.step += 1
        if self.count == 0:
            return
        import ctypes
        arr = (ctypes.c_double * 6)(*[float(x) for x in lrs])
        variant = self.adam_variant
        if variant == "auto":
            variant = "rows" if (self.device.type == "cuda" and adam_rows_agrees(self.device)) else "units"
        common = (self.device, self.params, self.grads, self.exp_avg, self.exp_avg_sq, self.count, self.cap, arr, float(beta1),
                  float(beta2), float(eps), self.step, 1 if zero_grad else 0, skip, self.touched if zero_grad else None,
                  self.active if zero_grad else None)
        if variant == "rows":
            if self._live_list is None or self._live_list.numel() < self.cap:  # scratch of the row-block kernels
                self._live_list = torch.empty(self.cap, dtype=torch.int32, device=self.device)
                self._live_count = torch.zeros(1, dtype=torch.int32, device=self.device)
            native.call("adam_rows", *common, self._live_list, self._live_count)
        else:
            native.call("adam", *common)
        if zero_grad:
            self.touched.zero_()
        else:
            self.active[:self.count] = 1  # dense update: every row may have moments now

    def mark_active(self):
        """Declare that Adam moments were written outside the optimiser kernel (e.g. loaded from a file)."""
        self.active[:self.count] = 1

    def mark_touched(self, index: torch.Tensor | None = None):
        """Declare that gradient rows were written outside the render kernels (all rows when ``index`` is None)."""
        if index is None:
            self.touched[:self.count] = 1
        else:
            self.touched[index] = 1

    def zero_grad(self):
        self.grads.zero_()
        self.touched.zero_()

    # -- optimiser state files ------------------------------------------------------------------
    def optimizer_state_dict(self, lrs=None) -> dict:
        """``torch.optim.Adam.state_dict()``-shaped dict with the reference's seven groups
        (xyz, f_dc, f_rest, opacity, scaling, rotation, means2D_meta; ``gaussian_nn_module.py:434-444``)."""
        n = self.count
        m, v = self.views("exp_avg"), self.views("exp_avg_sq")
        sh_m, sh_v = m["sh"].view(n, 16, 3), v["sh"].view(n, 16, 3)
        entries = [
            (m["xyz"], v["xyz"]), (sh_m[:, :1], sh_v[:, :1]), (sh_m[:, 1:], sh_v[:, 1:]), (m["opacity"], v["opacity"]),
            (m["scale"], v["scale"]), (m["rot"], v["rot"]),
        ]
        names = ["xyz", "f_dc", "f_rest", "opacity", "scaling", "rotation", "means2D_meta"]
        state = {}
        for i, (a, b) in enumerate(entries):
            state[i] = {"step": torch.tensor(float(self.step)), "exp_avg": a.detach().cpu().clone().contiguous(),
                        "exp_avg_sq": b.detach().cpu().clone().contiguous()}
        lr_map = {}
        if lrs is not None:
            lr_map = {"xyz": lrs[0], "f_dc": lrs[1], "f_rest": lrs[2], "scaling": lrs[3], "rotation": lrs[4],
                      "opacity": lrs[5], "means2D_meta": 0.0}
        groups = [{"lr": float(lr_map.get(nm, 0.0)), "name": nm, "betas": (0.9, 0.999), "eps": 1e-15, "weight_decay": 0,
                   "amsgrad": False, "params": [i]} for i, nm in enumerate(names)]
        return {"state": state, "param_groups": groups}

    def load_optimizer_state_dict(self, sd: dict):
        st = sd["state"]
        name_of = {g["params"][0]: g.get("name", str(i)) for i, g in enumerate(sd["param_groups"])}
        n = self.count
        m, v = self.views("exp_avg"), self.views("exp_avg_sq")
        for idx, entry in st.items():
            nm = name_of.get(idx, "")
            a, b = entry["exp_avg"].to(self.device), entry["exp_avg_sq"].to(self.device)
            if a.shape[0] != n:
                continue
            if nm == "xyz":
                m["xyz"].copy_(a); v["xyz"].copy_(b)
            elif nm == "f_dc":
                m["sh"].view(n, 16, 3)[:, :1].copy_(a.view(n, 1, 3)); v["sh"].view(n, 16, 3)[:, :1].copy_(b.view(n, 1, 3))
            elif nm == "f_rest":
                k = a.view(n, -1, 3).shape[1]
                m["sh"].view(n, 16, 3)[:, 1:1 + k].copy_(a.view(n, k, 3)); v["sh"].view(n, 16, 3)[:, 1:1 + k].copy_(b.view(n, k, 3))
            elif nm == "opacity":
                m["opacity"].copy_(a.view(n, 1)); v["opacity"].copy_(b.view(n, 1))
            elif nm == "scaling":
                m["scale"].copy_(a); v["scale"].copy_(b)
            elif nm == "rotation":
                m["rot"].copy_(a); v["rot"].copy_(b)
            if "step" in entry:
                self.step = int(float(entry["step"]))
        self.mark_active()
