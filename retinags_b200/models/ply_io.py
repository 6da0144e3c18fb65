"""Binary PLY reading/writing without third-party packages.

File layout of a Gaussian model (identical to vanilla 3DGS and to the reference,
``scene/gaussian_nn_module.py:480-513``): one ``vertex`` element of little-endian ``float``
properties ``x y z nx ny nz f_dc_0..2 f_rest_0..(3*(deg+1)^2-4) opacity scale_0..2 rot_0..3``; values
are raw (log-scale, logit-opacity, unnormalised w-x-y-z quaternion); ``f_rest`` is channel-major
(all red coefficients, then green, then blue) whereas the in-memory SH block is coefficient-major.

Point clouds used for initialisation (``scene/dataset_readers.py:148-181``) carry
``x y z nx ny nz red green blue`` with ``uchar`` colours.
"""
from __future__ import annotations

import numpy as np
import torch

_PLY_TYPES = {
    "char": "i1", "int8": "i1", "uchar": "u1", "uint8": "u1", "short": "i2", "int16": "i2", "ushort": "u2",
    "uint16": "u2", "int": "i4", "int32": "i4", "uint": "u4", "uint32": "u4", "float": "f4", "float32": "f4",
    "double": "f8", "float64": "f8",
}


def _parse_header(f, path: str):
    """(format, elements) of an open PLY file; the file position is left at the first byte of the data."""
    if f.readline().strip() != b"ply":
        raise ValueError(f"{path}: not a PLY file")
    fmt, elements, cur = None, [], None
    while True:
        line = f.readline()
        if not line:
            raise ValueError(f"{path}: truncated header")
        tok = line.decode("ascii", "replace").split()
        if not tok:
            continue
        if tok[0] == "format":
            fmt = tok[1]
        elif tok[0] == "element":
            cur = {"name": tok[1], "count": int(tok[2]), "props": []}
            elements.append(cur)
        elif tok[0] == "property":
            if tok[1] == "list":
                cur["props"].append(("list", tok[2], tok[3], tok[4]))
            else:
                cur["props"].append((tok[2], _PLY_TYPES[tok[1]]))
        elif tok[0] == "end_header":
            break
    return fmt, elements


def read_ply_vertices(path: str) -> np.ndarray:
    """Structured array of the ``vertex`` element of a PLY file (binary little/big endian or ascii)."""
    with open(path, "rb") as f:
        fmt, elements = _parse_header(f, path)
        endian = "<" if fmt in ("binary_little_endian", "ascii") else ">"
        for el in elements:
            if any(p[0] == "list" for p in el["props"]):
                if el["name"] == "vertex":
                    raise ValueError("list properties on the vertex element are not supported")
                break
            dtype = np.dtype([(n, endian + t) for n, t in el["props"]])
            if fmt == "ascii":
                rows = [f.readline().split() for _ in range(el["count"])]
                arr = np.zeros(el["count"], dtype=dtype)
                for j, (n, _) in enumerate(el["props"]):
                    arr[n] = [r[j] for r in rows]
            else:
                arr = np.frombuffer(f.read(dtype.itemsize * el["count"]), dtype=dtype, count=el["count"])
            if el["name"] == "vertex":
                return arr
    raise ValueError(f"{path}: no vertex element")


class PlyVertexStream:
    """The ``vertex`` element of a binary PLY file read piecewise through a memory map: a model of hundreds of
    millions of Gaussians (54 GB at 217 M) is walked in chunks of a few hundred MB instead of being parsed into host
    memory at once (the reference parses the whole file on rank 0, ``scene/gaussian_nn_module.py:134-174``).
    Only a leading vertex element of fixed-size properties is supported, which is what every Gaussian model file is."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            fmt, elements = _parse_header(f, path)
            self.offset = f.tell()
        if fmt not in ("binary_little_endian", "binary_big_endian"):
            raise ValueError(f"{path}: streaming needs a binary PLY file")
        el = elements[0] if elements else None
        if el is None or el["name"] != "vertex" or any(p[0] == "list" for p in el["props"]):
            raise ValueError(f"{path}: the first element must be a vertex element of scalar properties")
        endian = "<" if fmt == "binary_little_endian" else ">"
        self.dtype = np.dtype([(n, endian + t) for n, t in el["props"]])
        self.count = el["count"]
        self.names = self.dtype.names

    def memmap(self) -> np.ndarray:
        if self.count == 0:
            return np.zeros(0, dtype=self.dtype)
        return np.memmap(self.path, dtype=self.dtype, mode="r", offset=self.offset, shape=(self.count,))

    def chunks(self, rows: int = 2_000_000, start: int = 0, step: int = 1):
        """Yields (first row, structured array copy) for chunk ``start``, ``start + step``, ... of ``rows`` rows."""
        mm = self.memmap()
        nchunks = (self.count + rows - 1) // rows
        for k in range(start, nchunks, step):
            a = k * rows
            yield a, np.array(mm[a:min(self.count, a + rows)])  # one copy into host memory, then the pages can go
        del mm


def write_ply_vertices(path: str, names: list[str], data: np.ndarray, types: list[str] | None = None):
    """Write an (N, len(names)) array as binary little-endian PLY; ``types`` are PLY type names."""
    types = types or ["float"] * len(names)
    dtype = np.dtype([(n, "<" + _PLY_TYPES[t]) for n, t in zip(names, types)])
    out = np.empty(data.shape[0], dtype=dtype)
    for j, n in enumerate(names):
        out[n] = data[:, j]
    header = "ply\nformat binary_little_endian 1.0\n" + f"element vertex {data.shape[0]}\n" + \
        "".join(f"property {t} {n}\n" for n, t in zip(names, types)) + "end_header\n"
    with open(path, "wb") as f:
        f.write(header.encode("ascii"))
        f.write(out.tobytes())


def gaussian_attribute_names(sh_degree: int = 3) -> list[str]:
    n_rest = 3 * ((sh_degree + 1) ** 2 - 1)
    return (["x", "y", "z", "nx", "ny", "nz"] + [f"f_dc_{i}" for i in range(3)] + [f"f_rest_{i}" for i in range(n_rest)]
            + ["opacity"] + [f"scale_{i}" for i in range(3)] + [f"rot_{i}" for i in range(4)])


def _gaussian_rows(g: dict, sh_degree: int) -> np.ndarray:
    """(n, 62 at SH-3) float32 rows in file order from a dict of raw parameter tensors."""
    P = g["xyz"].shape[0]
    nc = (sh_degree + 1) ** 2
    sh = g["sh"].detach().cpu().float().view(P, 16, 3)
    f_dc = sh[:, 0]
    f_rest = sh[:, 1:nc].transpose(1, 2).reshape(P, -1)  # channel-major
    cols = [g["xyz"].detach().cpu().float(), torch.zeros(P, 3), f_dc, f_rest, g["opacity"].detach().cpu().float().view(P, 1),
            g["scale"].detach().cpu().float(), g["rot"].detach().cpu().float()]
    return torch.cat(cols, dim=1).numpy()


def _gaussian_header(count: int, sh_degree: int) -> bytes:
    names = gaussian_attribute_names(sh_degree)
    return ("ply\nformat binary_little_endian 1.0\n" + f"element vertex {count}\n" +
            "".join(f"property float {n}\n" for n in names) + "end_header\n").encode("ascii")


def save_gaussians(path: str, g: dict, sh_degree: int = 3, chunk: int = 2_000_000):
    """``g``: xyz (P,3), sh (P,48) coefficient-major, scale (P,3), rot (P,4), opacity (P,1) raw values. The rows are
    converted and written ``chunk`` at a time, so that the host never holds a second copy of a large sub-model."""
    P = int(g["xyz"].shape[0])
    with open(path, "wb") as f:
        f.write(_gaussian_header(P, sh_degree))
        for a in range(0, P, chunk):
            part = {k: v[a:a + chunk] for k, v in g.items()}
            f.write(np.ascontiguousarray(_gaussian_rows(part, sh_degree), dtype="<f4").tobytes())


def merge_gaussian_files(out_path: str, files: list[str], sh_degree: int = 3, block_rows: int = 1_000_000) -> int:
    """Concatenate Gaussian model files into one (``scene/gaussian_nn_module.py:58-132``: the whole-model merge)
    without loading them: files in this writer's layout are copied as bytes block by block, others are converted
    chunk by chunk. Returns the number of Gaussians written."""
    streams = [PlyVertexStream(f) for f in files]
    total = sum(st.count for st in streams)
    target = np.dtype([(n, "<f4") for n in gaussian_attribute_names(sh_degree)])
    with open(out_path, "wb") as out:
        out.write(_gaussian_header(total, sh_degree))
        for st in streams:
            if st.dtype == target:
                with open(st.path, "rb") as src:
                    src.seek(st.offset)
                    left = st.count * target.itemsize
                    while left > 0:
                        buf = src.read(min(left, block_rows * target.itemsize))
                        if not buf:
                            raise ValueError(f"{st.path}: truncated vertex data")
                        out.write(buf)
                        left -= len(buf)
            else:
                for _, v in st.chunks(block_rows):
                    out.write(np.ascontiguousarray(_gaussian_rows(gaussians_from_vertices(v, sh_degree), sh_degree), dtype="<f4").tobytes())
    return total


def gaussians_from_vertices(v: np.ndarray, max_sh_degree: int = 3) -> dict:
    """Parameter tensors of a structured vertex array (any property order, any SH degree up to 3)."""
    names = v.dtype.names
    P = v.shape[0]

    def col(n):
        return torch.from_numpy(np.ascontiguousarray(v[n]).astype(np.float32))

    xyz = torch.stack([col("x"), col("y"), col("z")], 1)
    sh = torch.zeros(P, 16, 3)
    sh[:, 0] = torch.stack([col(f"f_dc_{i}") for i in range(3)], 1)
    rest = sorted((n for n in names if n.startswith("f_rest_")), key=lambda s: int(s.split("_")[-1]))
    if rest:
        k = len(rest) // 3
        r = torch.stack([col(n) for n in rest], 1).view(P, 3, k).transpose(1, 2)  # -> (P,k,3)
        k = min(k, (max_sh_degree + 1) ** 2 - 1, 15)
        sh[:, 1:1 + k] = r[:, :k]
    scale = torch.stack([col(n) for n in sorted((n for n in names if n.startswith("scale_")), key=lambda s: int(s.split("_")[-1]))], 1)
    rot = torch.stack([col(n) for n in sorted((n for n in names if n.startswith("rot")), key=lambda s: int(s.split("_")[-1]))], 1)
    return dict(xyz=xyz.contiguous(), sh=sh.view(P, 48).contiguous(), scale=scale.contiguous(), rot=rot.contiguous(),
                opacity=col("opacity").view(P, 1).contiguous())


def load_gaussians(path: str, max_sh_degree: int = 3) -> dict:
    """Inverse of :func:`save_gaussians`; accepts any property order and lower SH degrees."""
    return gaussians_from_vertices(read_ply_vertices(path), max_sh_degree)


def iter_gaussians(path: str, max_sh_degree: int = 3, rows: int = 2_000_000, start: int = 0, step: int = 1):
    """Yields (first row, parameter dict) for chunks ``start``, ``start + step``, ... of a model file (memory-mapped)."""
    for a, v in PlyVertexStream(path).chunks(rows, start, step):
        yield a, gaussians_from_vertices(v, max_sh_degree)


def fetch_point_cloud(path: str, sample_rate: int = 1, seed: int = 0):
    """(points (N,3) float32, colors (N,3) float32 in [0,1], normals (N,3)) of an initialisation cloud;
    ``sample_rate`` N keeps a random 1/N subset (``scene/dataset_readers.py:148-164``)."""
    v = read_ply_vertices(path)
    names = v.dtype.names
    pts = np.stack([v["x"], v["y"], v["z"]], 1).astype(np.float32)
    if all(n in names for n in ("red", "green", "blue")):
        col = np.stack([v["red"], v["green"], v["blue"]], 1).astype(np.float32) / 255.0
    else:
        col = np.full_like(pts, 0.5)
    nrm = np.stack([v["nx"], v["ny"], v["nz"]], 1).astype(np.float32) if "nx" in names else np.zeros_like(pts)
    if sample_rate > 1:
        keep = np.random.default_rng(seed).permutation(pts.shape[0])[: pts.shape[0] // sample_rate]
        pts, col, nrm = pts[keep], col[keep], nrm[keep]
    return pts, col, nrm


def store_point_cloud(path: str, xyz: np.ndarray, rgb: np.ndarray):
    """Write ``x y z nx ny nz red green blue`` (``scene/dataset_readers.py:166-181``)."""
    n = xyz.shape[0]
    data = np.concatenate([xyz.astype(np.float32), np.zeros((n, 3), np.float32), rgb.astype(np.float32)], 1)
    write_ply_vertices(path, ["x", "y", "z", "nx", "ny", "nz", "red", "green", "blue"], data,
                       ["float"] * 6 + ["uchar"] * 3)
