"""ctypes binding of the native libraries (``librgs_cpu.so`` / ``librgs_cuda.so``).

Every entry point exists twice with the same argument list: ``rgs_cpu_<name>`` works on host
pointers, ``rgs_cuda_<name>`` on device pointers and takes the CUDA stream as its last argument
(the CPU twin ignores it).  :func:`call` picks the twin from the device of the tensors involved.
On a machine with a GPU the CUDA library is mandatory: a missing ``librgs_cuda.so`` raises instead
of silently falling back to another implementation.

Counterpart in the reference: the pybind extension
``rasterization_kernels/diff-gaussian-rasterization-half-gaussian/ext.cpp:15-19``.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

from .. import _build

_LOCK = threading.Lock()
_LIBS: dict[str, ctypes.CDLL] = {}

# signature alphabet: p = pointer, i = int64, f = double
SIGNATURES = {
    "project_emit": "ppipppippippp",
    "sort_ranges": "ppppipippp",
    "project_slots": "ppipppipppppp",
    "project_slots2": "ppipipppipppppp",
    "bin_instances": "pppppippppppppipiippp",
    "blend_fwd": "ppppppppp",
    "blend_fwd_push": "ppppppppipppp",
    "blend_bwd": "pppppppppp",
    "blend_bwd_depth": "ppppppppppp",
    "geom_bwd": "ppipppppip",
    "scatter_radii": "pppiipp",
    "adam": "ppppiipfffiipppp",
    "adam_rows": "ppppiipfffiipppppp",
    "composite_fwd": "pipiiiippp",
    "composite_bwd": "ppipiiiipip",
    "ssim_fwd": "ppiiiiiippp",
    "ssim_bwd": "pppiiiiiiffpp",
    "densify_classify": "piipppppppp",
    "densify_gather": "pppiippppppiipp",
    "records_pack": "pppipiipp",
    "records_unpack": "pipppiip",
}

_CTYPE = {"p": ctypes.c_void_p, "i": ctypes.c_int64, "f": ctypes.c_double}


class RgsCamera(ctypes.Structure):
    """Mirror of ``struct RgsCamera`` (csrc/rgs_math.h)."""

    _fields_ = [
        ("view", ctypes.c_float * 16),
        ("proj", ctypes.c_float * 16),
        ("c2w", ctypes.c_float * 16),
        ("campos", ctypes.c_float * 3),
        ("tan_fovx", ctypes.c_float),
        ("tan_fovy", ctypes.c_float),
        ("focal_x", ctypes.c_float),
        ("focal_y", ctypes.c_float),
        ("W", ctypes.c_int),
        ("H", ctypes.c_int),
        ("tiles_x", ctypes.c_int),
        ("tiles_y", ctypes.c_int),
        ("box_lo", ctypes.c_float * 3),
        ("box_hi", ctypes.c_float * 3),
        ("bg", ctypes.c_float * 3),
        ("sh_degree", ctypes.c_int),
        ("scale_modifier", ctypes.c_float),
        ("raw_params", ctypes.c_int),
        ("tight_rect", ctypes.c_int),
    ]


class RgsSegment(ctypes.Structure):
    """Mirror of ``struct RgsSegment`` (csrc/rgs_api.h)."""

    _fields_ = [(n, ctypes.c_void_p) for n in (
        "xyz", "sh", "scale", "rot", "opacity", "g_xyz", "g_sh", "g_scale", "g_rot", "g_opacity",
        "g_mean2d", "stat_grad", "stat_denom", "stat_maxrad", "touched")] + [("count", ctypes.c_int64)]


class RgsDensifyCfg(ctypes.Structure):
    """Mirror of ``struct RgsDensifyCfg`` (csrc/rgs_surgery.h)."""

    _fields_ = [("max_grad", ctypes.c_float), ("dense_extent", ctypes.c_float), ("min_opacity", ctypes.c_float),
                ("max_screen", ctypes.c_float), ("world_max", ctypes.c_float), ("skip_clone", ctypes.c_int),
                ("skip_split", ctypes.c_int), ("skip_prune", ctypes.c_int), ("no_grow", ctypes.c_int),
                ("seed", ctypes.c_uint64)]


SURGERY_BLOCK = 1024

CNT_VIS, CNT_INST, CNT_OVERFLOW, CNT_STATUS, CNT_WORDS = 0, 1, 2, 3, 8
CNT_INST2 = 5  # instances of the far slab (two-slab binning)
SPLAT_FLOATS = 12


def cuda_required() -> bool:
    return torch.cuda.is_available()


def lib(kind: str) -> ctypes.CDLL:
    """Load (building first when stale) ``librgs_<kind>.so``; kind is "cpu" or "cuda"."""
    with _LOCK:
        if kind in _LIBS:
            return _LIBS[kind]
        if kind == "cpu":
            path = _build.build_cpu()
        elif kind == "cuda":
            path = _build.LIB / "librgs_cuda.so"
            if not path.exists() or _build._stale(path, [_build.CSRC / s for s in _build.CUDA_SOURCES
                                                          if (_build.CSRC / s).exists()]):
                path = _build.build_cuda()
        else:
            raise ValueError(kind)
        handle = ctypes.CDLL(str(path))
        _LIBS[kind] = handle
        return handle


def _fn(kind: str, name: str, sig: str | None = None):
    handle = lib(kind)
    full = f"rgs_{kind}_{name}"
    fn = getattr(handle, full)
    if not getattr(fn, "_rgs_ready", False):
        sig = sig if sig is not None else SIGNATURES[name]
        fn.argtypes = [_CTYPE[c] for c in sig]
        fn.restype = ctypes.c_int
        fn._rgs_ready = True
    return fn


def ptr(x):
    """Raw address of a tensor / ctypes object / None."""
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x.data_ptr()
    if isinstance(x, (ctypes.Structure, ctypes.Array)):
        return ctypes.addressof(x)
    if isinstance(x, int):
        return x
    raise TypeError(type(x))


def stream_ptr(device: torch.device):
    if device.type != "cuda":
        return None
    return torch.cuda.current_stream(device).cuda_stream


# kernels launched by one call of an entry point (the radix sort's count depends on the tile count)
_KERNELS = {"project_slots": 1, "project_slots2": 2, "project_slots2_geom": 2, "colour_slab": 1, "tile_maps_or": 1, "tile_map_push": 1, "project_emit": 1, "blend_fwd": 1, "blend_bwd": 1, "geom_bwd": 1, "scatter_radii": 1, "adam": 1, "adam_rows": 2,
            "composite_fwd": 1, "composite_bwd": 1, "ssim_fwd": 1, "ssim_bwd": 1, "densify_classify": 2, "blend_fwd_slab": 1, "blend_bwd_slab": 1}
_LAUNCHES = [0]
_SORT_SWEEP = [os.environ.get("RGS_SORT", "") != "3k"]


def _sort_launches(passes: int) -> int:
    """Kernels of one radix sort of the binning: digit counts + one scatter per pass, or three kernels per pass."""
    return 1 + passes if _SORT_SWEEP[0] else 3 * passes


def cuda_switch(name: str, on: bool) -> bool:
    """Flip a run-time switch of the CUDA library and return the setting that was in force.

    ``loss_cluster``: the fused composite + SSIM forward runs as 2 x 2 thread-block clusters that share the rims of
    their windows through distributed shared memory (off, the default: every block composites its whole window).
    ``sort_sweep``: the radix sort of the binning counts the digits of all passes up front and scatters with a
    decoupled look-back (off: histogram, scan and scatter launches per pass).
    """
    fn = getattr(lib("cuda"), f"rgs_cuda_{name}")
    fn.argtypes = [ctypes.c_int]
    fn.restype = ctypes.c_int
    if name == "sort_sweep":
        _SORT_SWEEP[0] = bool(on)
    return bool(fn(1 if on else 0))


def launch_count() -> int:
    """Number of kernels of the CUDA library launched so far by this process."""
    return _LAUNCHES[0]


def _count_launches(name: str, args) -> int:
    if name == "sort_ranges":
        tiles = max(int(args[6]), 1)
        bits = 32 + max(tiles - 1, 0).bit_length()
        return 3 * ((bits + 7) // 8) + 1
    if name == "bin_instances":
        tiles = max(int(args[17]), 1)
        if tiles <= 14336 and os.environ.get("RGS_TILE_GROUPING", "") == "count":
            return _sort_launches(4) + 2 + 4  # depth sort, instance count + scan, segmented counting (count, 2 scans, emit)
        return _sort_launches(4) + 3 + _sort_launches(max(1, (max(tiles - 1, 0).bit_length() + 7) // 8)) + 1
    if name == "bin_slab":
        tiles, slab, filtered = max(int(args[16]), 1), int(args[20]), args[22] is not None
        n = _sort_launches(4) if slab == 0 else 0  # depth order of the visible splats, shared by both slabs
        n += 2 if filtered else 0  # summed-area table of the open tiles + filtered instance counts
        n += 3  # instance counts per segment, their scan, emission
        return n + _sort_launches(max(1, (max(tiles - 1, 0).bit_length() + 7) // 8)) + 1  # tile sort + tile ranges
    return _KERNELS.get(name, 1)


def call(name: str, device: torch.device, *args, sig: str | None = None) -> None:
    """Invoke ``rgs_<cpu|cuda>_<name>(*args, stream)`` and raise on a non-zero status."""
    kind = "cuda" if device.type == "cuda" else "cpu"
    if kind == "cuda":
        _LAUNCHES[0] += _count_launches(name, args)
    fn = _fn(kind, name, sig)
    conv = []
    for a in args:
        if isinstance(a, (torch.Tensor, ctypes.Structure, ctypes.Array)) or a is None:
            conv.append(ptr(a))
        else:
            conv.append(a)
    if kind == "cuda":
        with torch.cuda.device(device):
            rc = fn(*conv, stream_ptr(device))
    else:
        rc = fn(*conv, None)
    if rc != 0:
        raise RuntimeError(f"rgs_{kind}_{name} failed with status {rc}")


def pointer_array(tensors) -> ctypes.Array:
    """Host array of raw addresses (for entry points that take a list of buffers)."""
    arr = (ctypes.c_void_p * max(len(tensors), 1))()
    for i, t in enumerate(tensors):
        arr[i] = ptr(t)
    return arr
