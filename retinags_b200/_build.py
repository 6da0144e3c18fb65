"""In-tree build of the native libraries.

``librgs_cpu.so`` (g++/OpenMP) and ``librgs_cuda.so`` (nvcc, sm_100a only) are written to
``retinags_b200/lib/``.  The reference builds its single extension through
``rasterization_kernels/diff-gaussian-rasterization-half-gaussian/setup.py:26-34`` with no
architecture flags at all; here the architecture is fixed to Blackwell (``compute_100a``).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"

CPU_SOURCES = ["rgs_cpu.cpp"]
CUDA_SOURCES = [
    "rgs_raster.cu",
    "rgs_sort.cu",
    "rgs_binning.cu",
    "rgs_loss.cu",
    "rgs_model.cu",
    "rgs_p2p.cu",
    "rgs_border.cu",
    "rgs_aux.cu",
    "rgs_surgery.cu",
    "rgs_ssim_tc.cu",
    "rgs_noalloc.cu",
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _digest(paths) -> str:
    h = hashlib.sha1()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _headers():
    return sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))


def _stale(target: Path, sources) -> bool:
    stamp = target.with_suffix(".sha1")
    if not target.exists() or not stamp.exists():
        return True
    return stamp.read_text().strip() != _digest(list(sources) + _headers())


def _run(cmd, log: Path | None = None):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(" ".join(map(str, cmd)) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError(f"native build failed: {' '.join(map(str, cmd))}")
    return proc.stdout


def build_cpu(force: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    target = LIB / "librgs_cpu.so"
    sources = [CSRC / s for s in CPU_SOURCES if (CSRC / s).exists()]
    if force or _stale(target, sources):
        tmp = target.with_suffix(f".tmp{os.getpid()}.so")
        _run(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-I", str(CSRC), "-o", str(tmp)]
             + [str(s) for s in sources])
        os.replace(tmp, target)
        target.with_suffix(".sha1").write_text(_digest(sources + _headers()))
    return target


def nvcc_path() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def build_cuda(force: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    target = LIB / "librgs_cuda.so"
    sources = [CSRC / s for s in CUDA_SOURCES if (CSRC / s).exists()]
    if force or _stale(target, sources):
        nvcc = nvcc_path()
        if nvcc is None:
            raise RuntimeError("nvcc not found: cannot build librgs_cuda.so")
        objs = []
        obj_dir = LIB / "obj"
        obj_dir.mkdir(exist_ok=True)
        procs = []
        for s in sources:
            o = obj_dir / (s.stem + ".o")
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)]
            procs.append((s, o, cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        for s, o, cmd, pr in procs:
            out, _ = pr.communicate()
            (obj_dir / (s.stem + ".ptxas.log")).write_text(" ".join(cmd) + "\n" + out)
            if pr.returncode != 0:
                sys.stderr.write(out)
                raise RuntimeError(f"nvcc failed on {s.name}")
            objs.append(o)
        tmp = target.with_suffix(f".tmp{os.getpid()}.so")
        _run([nvcc, "-shared", "-o", str(tmp)] + [str(o) for o in objs] + ["-lcudart"])
        os.replace(tmp, target)
        target.with_suffix(".sha1").write_text(_digest(sources + _headers()))
    return target


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_cpu(force))
    if "--cpu-only" not in sys.argv:
        print(build_cuda(force))
