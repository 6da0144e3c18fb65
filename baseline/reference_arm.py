"""Reference arm of ``bench.py``: the unmodified reference trainer on the benchmark's synthetic scene.

What runs: ``main.py`` of the reference (a byte-for-byte copy under ``baseline/_ref/reference_src``)
through its own ``Trainer4TreePartition.train()`` and its own CUDA extension
(``diff_gaussian_rasterization_half_gaussian``, built unmodified for sm_100 into ``baseline/_ref``).
Nothing of this repository's models, kernels or engine is on that path.  What this file adds around it:

* import shims for third-party packages that the image lacks and the timed path never executes
  (``plyfile`` reader/writer; ``simple_knn._C.distCUDA2`` and the vanilla ``diff_gaussian_rasterization``,
  which are empty git submodules in the reference; ``lpipsPyTorch`` weight download) -- written to
  ``baseline/_ref/shims``;
* the scene on disk: Blender-layout cameras + PNG targets and a vanilla-3DGS ``point_cloud.ply`` holding
  the very Gaussians of the own arm (same seeded generator), which the reference loads with
  ``--ply_iteration``;
* timing: the reference writes one TensorBoard record per iteration (``iter_time``); the wall-clock
  stamps of those records bracket whole iterations (data loading, forward, backward, optimiser step), so
  K steps take ``stamp[W+K] - stamp[W]``; the maximum over ranks is reported.  The reference's own
  ``iter_time`` value excludes the optimiser step and is therefore not used.
"""
from __future__ import annotations

import glob
import json
import os
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SRC = os.path.join(REF, "reference_src")
SHIMS = os.path.join(REF, "shims")
# checkout of the reference to copy from when baseline/_ref/reference_src does not exist yet
UPSTREAM = os.environ.get("RGS_REFERENCE_SRC", os.path.join(os.path.dirname(REF), "..", "..", "reference"))

PLYFILE_SHIM = '''"""Minimal stand-in for the ``plyfile`` package (binary little-endian vertex elements only)."""
import numpy as np

_T = {"char": "i1", "uchar": "u1", "short": "i2", "ushort": "u2", "int": "i4", "uint": "u4", "float": "f4", "double": "f8",
      "int8": "i1", "uint8": "u1", "int16": "i2", "uint16": "u2", "int32": "i4", "uint32": "u4", "float32": "f4", "float64": "f8"}
_R = {"i1": "char", "u1": "uchar", "i2": "short", "u2": "ushort", "i4": "int", "u4": "uint", "f4": "float", "f8": "double"}


class PlyProperty:
    def __init__(self, name, dtype):
        self.name, self.dtype = name, dtype


class PlyElement:
    def __init__(self, name, data):
        self.name, self.data = name, data
        self.properties = [PlyProperty(n, data.dtype[n]) for n in data.dtype.names]

    @staticmethod
    def describe(data, name):
        return PlyElement(name, data)

    def __getitem__(self, key):
        return self.data[key]

    @property
    def count(self):
        return self.data.shape[0]


class PlyData:
    def __init__(self, elements):
        self.elements = list(elements)

    def __getitem__(self, name):
        for e in self.elements:
            if e.name == name:
                return e
        raise KeyError(name)

    @staticmethod
    def read(path):
        with open(path, "rb") as f:
            assert f.readline().strip() == b"ply"
            elements, cur = [], None
            while True:
                tok = f.readline().decode("ascii").split()
                if not tok:
                    continue
                if tok[0] == "element":
                    cur = [tok[1], int(tok[2]), []]
                    elements.append(cur)
                elif tok[0] == "property":
                    cur[2].append((tok[2], "<" + _T[tok[1]]))
                elif tok[0] == "end_header":
                    break
            out = []
            for name, count, props in elements:
                dt = np.dtype(props)
                out.append(PlyElement(name, np.fromfile(f, dtype=dt, count=count)))
        return PlyData(out)

    def write(self, path):
        with open(path, "wb") as f:
            hdr = "ply\\nformat binary_little_endian 1.0\\n"
            for e in self.elements:
                hdr += "element %s %d\\n" % (e.name, e.data.shape[0])
                for n in e.data.dtype.names:
                    hdr += "property %s %s\\n" % (_R[e.data.dtype[n].str[1:]], n)
            hdr += "end_header\\n"
            f.write(hdr.encode("ascii"))
            for e in self.elements:
                e.data.astype(e.data.dtype.newbyteorder("<")).tofile(f)
'''

SIMPLE_KNN_SHIM = '''"""Stand-in for the absent ``simple_knn`` submodule: never called when training starts from a PLY."""
import torch


def distCUDA2(points):
    d = torch.cdist(points[:4096], points[:4096])
    raise RuntimeError("simple_knn is an empty submodule in the reference checkout; start from a point_cloud.ply")
'''

VANILLA_SHIM = '''"""Stand-in for the absent vanilla ``diff_gaussian_rasterization`` submodule (import-only in the trainer)."""
from typing import NamedTuple


class GaussianRasterizationSettings(NamedTuple):
    image_height: int = 0
    image_width: int = 0


class GaussianRasterizer:
    def __init__(self, *a, **k):
        raise RuntimeError("the vanilla rasterizer is an empty submodule in the reference checkout")
'''


def available() -> str | None:
    """None when the reference arm can run, else the reason (one line)."""
    ext = glob.glob(os.path.join(REF, "diff_gaussian_rasterization_half_gaussian", "_C*.so"))
    if not ext:
        return "reference CUDA extension not built under baseline/_ref (build it with TORCH_CUDA_ARCH_LIST=10.0 pip install --target baseline/_ref)"
    if not os.path.isdir(UPSTREAM) and not os.path.isdir(SRC):
        return "reference sources not present"
    return None


def prepare_tree():
    """Unmodified copy of the reference's Python tree + shims for packages the image lacks."""
    if not os.path.isdir(SRC):
        shutil.copytree(UPSTREAM, SRC, ignore=shutil.ignore_patterns(".git", "assets", "third_party", "*.so"))
    os.makedirs(SHIMS, exist_ok=True)
    try:
        import plyfile  # noqa: F401
    except ImportError:
        open(os.path.join(SHIMS, "plyfile.py"), "w").write(PLYFILE_SHIM)
    os.makedirs(os.path.join(SHIMS, "simple_knn"), exist_ok=True)
    open(os.path.join(SHIMS, "simple_knn", "__init__.py"), "w").write("")
    open(os.path.join(SHIMS, "simple_knn", "_C.py"), "w").write(SIMPLE_KNN_SHIM)
    os.makedirs(os.path.join(SHIMS, "diff_gaussian_rasterization"), exist_ok=True)
    open(os.path.join(SHIMS, "diff_gaussian_rasterization", "__init__.py"), "w").write(VANILLA_SHIM)


def write_scene(root: str, args, n_views: int, device):
    """Blender-layout dataset + ``<model>/point_cloud/iteration_1/point_cloud.ply`` with the own arm's Gaussians."""
    import numpy as np
    import torch

    sys.path.insert(0, os.path.dirname(HERE))
    from retinags_b200.bench_session import ClusterScene, chunks_of
    from retinags_b200.data import readers, synthetic
    from retinags_b200.models import ply_io
    from retinags_b200.ops.rasterize import RenderTask, Segment, make_camera

    data_dir, model_dir = os.path.join(root, "data"), os.path.join(root, "model")
    done = os.path.join(root, "READY")
    if os.path.exists(done):
        return data_dir, model_dir
    os.makedirs(data_dir, exist_ok=True)
    cams = synthetic.hemisphere_cameras(n_views, 8.0, args.width, args.height, 50.0, args.seed)
    gt = ClusterScene(args.seed + 1, device)
    parts = [gt.gaussians(m, k, 3) for k, m in chunks_of(args.gt_gaussians)]
    g = {name: torch.cat([p[name] for p in parts]) for name in parts[0]}
    seg = Segment(g["xyz"], g["sh"], g["scale"], g["rot"], g["opacity"])
    task = RenderTask(device)
    for cam in cams:
        out = task.forward(make_camera(cam, 3), [seg], check=True)
        cam.image = out[..., :3].permute(2, 0, 1).contiguous().cpu()
    pts = g["xyz"][:100000].cpu().numpy()
    readers.write_blender_scene(data_dir, cams, cams[:2], pts, np.full_like(pts, 128.0))
    del task, seg, g, parts
    torch.cuda.empty_cache()
    # the Gaussians of the own arm, chunk by chunk, in vanilla-3DGS vertex layout
    ply_dir = os.path.join(model_dir, "point_cloud", "iteration_1")
    os.makedirs(ply_dir, exist_ok=True)
    names = ply_io.gaussian_attribute_names(3)
    scene = ClusterScene(args.seed, device)
    with open(os.path.join(ply_dir, "point_cloud.ply"), "wb") as f:
        hdr = "ply\nformat binary_little_endian 1.0\n" + f"element vertex {args.gaussians}\n" + \
            "".join(f"property float {n}\n" for n in names) + "end_header\n"
        f.write(hdr.encode("ascii"))
        for k, m in chunks_of(args.gaussians):
            c = scene.gaussians(m, k, 3)
            sh = c["sh"].view(m, 16, 3)
            rows = torch.cat([c["xyz"], torch.zeros(m, 3, device=device), sh[:, 0], sh[:, 1:].transpose(1, 2).reshape(m, 45),
                              c["opacity"], c["scale"], c["rot"]], dim=1)
            f.write(rows.cpu().numpy().astype("<f4").tobytes())
    open(done, "w").write("ok")
    return data_dir, model_dir


def read_iteration_stamps(tb_dir: str, world: int):
    """Per rank: sorted (iteration, wall_time) of the ``iter_time`` scalars the reference logged."""
    from tensorboard.backend.event_processing.event_accumulator import EventAccumulator
    out = {}
    for r in range(world):
        files = glob.glob(os.path.join(tb_dir, f"rank_{r}", "events.out.tfevents.*"))
        stamps = []
        for fn in files:
            acc = EventAccumulator(fn, size_guidance={"scalars": 0})
            acc.Reload()
            if "iter_time" in acc.Tags().get("scalars", []):
                stamps += [(e.step, e.wall_time) for e in acc.Scalars("iter_time")]
        out[r] = sorted(stamps)
    return out


def main(args):
    why = available()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return
    world = args.gpus
    if int(os.environ.get("RANK", "0")) != 0:
        return  # launched under torchrun: rank 0 drives the reference's own torchrun below
    prepare_tree()
    n_iter = args.warmup + args.steps + 1
    n_views = n_iter * args.batch + 2 * args.batch
    root = os.environ.get("RGS_REF_WORKDIR", "/tmp/rgs_reference_arm") + f"_{args.gaussians}_{args.width}x{args.height}_{n_views}"
    data_dir, model_dir = os.path.join(root, "data"), os.path.join(root, "model")
    # the scene is written by a child process so that no CUDA context of this driver stays on GPU 0
    child_env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE")}
    wr = subprocess.run([sys.executable, os.path.abspath(__file__), "--write-scene", root, str(n_views), str(args.gaussians),
                         str(args.width), str(args.height), str(args.gt_gaussians), str(args.seed)], env=child_env,
                        capture_output=True, text=True)
    if wr.returncode != 0:
        print(json.dumps({"impl": "reference", "unavailable": ("could not write the synthetic scene: " + wr.stderr[-300:]).replace("\n", " | ")}),
              flush=True)
        return
    for d in glob.glob(os.path.join(model_dir, "rank_*")):
        shutil.rmtree(d, ignore_errors=True)
    depth = max(0, world.bit_length() - 1)
    max_load = 2 * args.batch
    if getattr(args, "bvh_depth", None) is not None and args.bvh_depth > depth:
        depth = args.bvh_depth  # more sub-models than GPUs: every camera costs one render task per local sub-model
        max_load = args.batch * max(1, (2 ** depth + world - 1) // world)
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([SHIMS, REF, SRC, env.get("PYTHONPATH", "")])
    # allocator hint that torch's own out-of-memory message recommends; the reference's code is untouched
    env.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_PORT", "MASTER_ADDR", "TORCHELASTIC_RUN_ID", "GROUP_RANK",
              "LOCAL_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE", "TORCHELASTIC_RESTART_COUNT",
              "TORCHELASTIC_MAX_RESTARTS", "TORCHELASTIC_USE_AGENT_STORE", "TORCH_NCCL_ASYNC_ERROR_HANDLING"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29800 + os.getpid() % 100), "main.py", "-s", data_dir, "-m", model_dir,
           "--bvh_depth", str(depth), "--MAX_BATCH_SIZE", str(args.batch), "--MAX_LOAD", str(max_load), "-r", "1",
           "--ply_iteration", "1", "--ENABLE_TENSORBOARD", "--logdir", os.path.join(root, "tb"), "--epochs", "1",
           "--iterations", str(n_views), "--EVAL_INTERVAL_EPOCH", "100000", "--SAVE_INTERVAL_EPOCH", "100000",
           "--densify_from_iter", "100000000", "--log_level", "30", "--DATALOADER_FIX_SEED"]
    tb_dir = os.path.join(root, "tb")
    shutil.rmtree(tb_dir, ignore_errors=True)
    log = open(os.path.join(root, "reference_run.log"), "w")
    proc = subprocess.Popen(cmd, cwd=SRC, env=env, stdout=log, stderr=subprocess.STDOUT)
    deadline = time.time() + float(os.environ.get("RGS_REF_TIMEOUT", "2400"))
    stamps, need = {}, args.warmup + args.steps + 1
    try:
        while time.time() < deadline:
            time.sleep(5.0)
            try:
                stamps = read_iteration_stamps(tb_dir, world)
            except Exception:
                stamps = {}
            if stamps and all(len(v) >= need for v in stamps.values()):
                break
            if proc.poll() is not None:
                stamps = read_iteration_stamps(tb_dir, world)
                break
    finally:
        if proc.poll() is None:  # enough iterations recorded: stop before the end-of-epoch save/eval
            proc.terminate()
            try:
                proc.wait(timeout=60)
            except subprocess.TimeoutExpired:
                proc.kill()
    log.close()
    if not stamps or not all(len(v) >= need for v in stamps.values()):
        dbg = ""
        for fn in sorted(glob.glob(os.path.join(SRC, "debugger", "debug_*.txt"))):
            txt = open(fn).read()
            if "Error" in txt or "error" in txt:
                dbg = txt[-400:].replace("\n", " | ")
        got = min((len(v) for v in stamps.values()), default=0)
        partial = ""
        if got >= 3:
            per = max((v[got - 1][1] - v[1][1]) / (got - 2) for v in stamps.values())
            partial = f" (the {got - 2} iterations it completed after the first took {1e3 * per:.0f} ms each)"
        print(json.dumps({"impl": "reference", "unavailable": f"the reference stopped after {got} of {need} iterations{partial}: {dbg}"[:900]}),
              flush=True)
        return
    W, K = args.warmup, args.steps
    per_rank = [v[W + K][1] - v[W][1] for v in stamps.values()]
    sec = max(per_rank)
    out = {"metric": "train views/s (62.9M GS, 1600x1036)", "value": K * args.batch / sec, "unit": "views/s", "n_gpus": world,
           "steps": K, "warmup": W, "ms_per_step": 1e3 * sec / K, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "reference",
           "config": {"model": "3DGS SH-3, seeded 64-cluster mixture in a 20-unit box", "gaussians": args.gaussians,
                      "global_batch": args.batch, "resolution": [args.width, args.height], "bvh_depth": depth,
                      "parallelism": f"spatial-mp{world}", "transport": "nccl send/recv (reference)",
                      "timing": "wall-clock stamps of the reference's own per-iteration TensorBoard records, max over ranks"},
           "e2e": {"value": K * args.batch / sec, "unit": "views/s", "note": "the reference loads PNG targets from disk through its DataLoader each step"},
           "gpu_launches": None}
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(HERE))
    if len(sys.argv) > 1 and sys.argv[1] == "--write-scene":
        import argparse
        import torch
        ns = argparse.Namespace(gaussians=int(sys.argv[4]), width=int(sys.argv[5]), height=int(sys.argv[6]),
                                gt_gaussians=int(sys.argv[7]), seed=int(sys.argv[8]))
        write_scene(sys.argv[2], ns, int(sys.argv[3]), torch.device("cuda", 0))
        sys.exit(0)
    import bench
    a = bench.parse_args()
    main(a)
