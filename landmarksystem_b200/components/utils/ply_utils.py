"""PLY point-cloud I/O and initial point clouds (reference:
landmark/nerf_components/utils/ply_utils.py:17-144).

The reference relies on the ``plyfile`` package; this module reads and writes the same files
(binary little-endian or ASCII, one ``vertex`` element with scalar properties) with numpy only.
"""
from __future__ import annotations

import os
from typing import Dict, List, Sequence, Tuple

import numpy as np

from .graphics_utils import BasicPointCloud

_PLY_TO_NP = {"float": "f4", "float32": "f4", "double": "f8", "float64": "f8", "uchar": "u1", "uint8": "u1",
              "char": "i1", "int8": "i1", "short": "i2", "int16": "i2", "ushort": "u2", "uint16": "u2", "int": "i4",
              "int32": "i4", "uint": "u4", "uint32": "u4"}
_NP_TO_PLY = {"f4": "float", "f8": "double", "u1": "uchar", "i1": "char", "i2": "short", "u2": "ushort", "i4": "int",
              "u4": "uint"}


def read_ply(path: str) -> np.ndarray:
    """Return the ``vertex`` element as a numpy structured array."""
    with open(path, "rb") as fh:
        assert fh.readline().strip() == b"ply", f"{path} is not a PLY file"
        fmt, count, props, in_vertex = None, 0, [], False
        while True:
            line = fh.readline().decode("ascii").strip()
            if line == "end_header":
                break
            tok = line.split()
            if not tok:
                continue
            if tok[0] == "format":
                fmt = tok[1]
            elif tok[0] == "element":
                in_vertex = tok[1] == "vertex"
                if in_vertex:
                    count = int(tok[2])
            elif tok[0] == "property" and in_vertex:
                assert tok[1] != "list", "list properties are not supported in the vertex element"
                props.append((tok[2], _PLY_TO_NP[tok[1]]))
        if fmt == "ascii":
            data = np.loadtxt(fh, max_rows=count, ndmin=2)
            out = np.empty(count, dtype=[(n, t) for n, t in props])
            for i, (n, _) in enumerate(props):
                out[n] = data[:, i]
            return out
        order = "<" if fmt == "binary_little_endian" else ">"
        dtype = np.dtype([(n, order + t) for n, t in props])
        return np.frombuffer(fh.read(count * dtype.itemsize), dtype=dtype, count=count).copy()


def write_ply(path: str, columns: Dict[str, np.ndarray], comments: Sequence[str] = ()) -> None:
    """Write equal-length 1-D arrays as the properties of a binary little-endian ``vertex`` element."""
    names = list(columns.keys())
    n = len(columns[names[0]]) if names else 0
    dtype = np.dtype([(k, "<" + np.asarray(columns[k]).dtype.newbyteorder("<").str[1:]) for k in names])
    data = np.empty(n, dtype=dtype)
    for k in names:
        data[k] = columns[k]
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as fh:
        header = ["ply", "format binary_little_endian 1.0"] + [f"comment {c}" for c in comments]
        header.append(f"element vertex {n}")
        header += [f"property {_NP_TO_PLY[dtype[k].str[1:]]} {k}" for k in names]
        header.append("end_header")
        fh.write(("\n".join(header) + "\n").encode("ascii"))
        fh.write(data.tobytes())


def fetchPly(path: str) -> BasicPointCloud:
    v = read_ply(path)
    pos = np.stack([v["x"], v["y"], v["z"]], 1).astype(np.float32)
    if "red" in v.dtype.names:
        col = np.stack([v["red"], v["green"], v["blue"]], 1).astype(np.float32) / 255.0
    else:
        col = np.full_like(pos, 0.5)
    if "nx" in v.dtype.names:
        nrm = np.stack([v["nx"], v["ny"], v["nz"]], 1).astype(np.float32)
    else:
        nrm = np.zeros_like(pos)
    return BasicPointCloud(points=pos, colors=col, normals=nrm)


def fetchLas(path: str) -> BasicPointCloud:
    """LAS point clouds need the external ``laspy`` package, which is not available offline."""
    try:
        import laspy
    except ImportError as exc:
        raise RuntimeError("reading .las point clouds requires the 'laspy' package") from exc
    las = laspy.read(path)
    pos = np.stack([las.x, las.y, las.z], 1).astype(np.float32)
    col = np.stack([las.red, las.green, las.blue], 1).astype(np.float32) / 65535.0
    return BasicPointCloud(points=pos, colors=col, normals=np.zeros_like(pos))


def storePly(path: str, xyz: np.ndarray, rgb: np.ndarray) -> None:
    xyz = np.asarray(xyz, dtype=np.float32)
    rgb = np.asarray(rgb)
    zeros = np.zeros(len(xyz), dtype=np.float32)
    write_ply(path, {"x": xyz[:, 0], "y": xyz[:, 1], "z": xyz[:, 2], "nx": zeros, "ny": zeros, "nz": zeros,
                     "red": rgb[:, 0].astype(np.uint8), "green": rgb[:, 1].astype(np.uint8),
                     "blue": rgb[:, 2].astype(np.uint8)})


def init_ply(datadir: str, aabb: Sequence[Sequence[float]], n_points=100_000, seed: int = 0, init_points_num=None):
    """Random cloud on the ground plane (``z = lb_z``) of the AABB, written to
    ``datadir/points3d_init.ply`` and returned as a path (the reference's fallback when no SfM cloud exists).

    The reference's form ``init_ply(folder, aabb, init_type, init_points_num)`` (ply_utils.py:17-50) is accepted as
    well and returns the cloud itself: ``init_type="ply"`` draws the random cloud, ``"colmap"`` reads
    ``folder/sparse/0/points3D.{ply,bin,txt}`` (converting to ``.ply`` on first use)."""
    if isinstance(n_points, str):
        kind, count = n_points, int(init_points_num if init_points_num is not None else (seed or 100_000))
        if kind == "colmap":
            from ..data.datasets.colmap_loader import read_points3D_binary, read_points3D_text

            base = os.path.join(datadir, "sparse", "0")
            ply = os.path.join(base, "points3D.ply")
            if not os.path.exists(ply):
                try:
                    xyz, rgb, _ = read_points3D_binary(os.path.join(base, "points3D.bin"))
                except FileNotFoundError:
                    xyz, rgb, _ = read_points3D_text(os.path.join(base, "points3D.txt"))
                storePly(ply, xyz, rgb)
            return fetchPly(ply)
        assert kind == "ply", f"init_type '{kind}' is not known (ply, colmap)"
        return fetchPly(init_ply(datadir, aabb, count))
    path = os.path.join(datadir, "points3d_init.ply")
    rng = np.random.default_rng(seed)
    lb, ub = np.asarray(aabb[0], dtype=np.float32), np.asarray(aabb[1], dtype=np.float32)
    xyz = rng.random((n_points, 3), dtype=np.float32) * (ub - lb) + lb
    xyz[:, 2] = lb[2]
    rgb = (rng.random((n_points, 3)) * 255).astype(np.uint8)
    storePly(path, xyz, rgb)
    return path


def get_pcd(config, aabb=None, *reference_tail, dataset=None) -> BasicPointCloud:
    """Initial cloud: ``config.point_path`` (.ply / .las) if given, else the sparse reconstruction of ``dataset`` when it
    carries one (COLMAP datasets, in the dataset's own world frame), else a random ground-plane cloud.

    The reference's form ``get_pcd(loaded_iter, config, aabb, logfolder, model)`` (ply_utils.py:116-144) is accepted:
    with ``loaded_iter`` set the model loads ``config.ckpt`` and nothing is returned, otherwise the cloud is built as
    above (COLMAP points for ``dataset_name="Colmap"``)."""
    if reference_tail or not (hasattr(config, "get") or hasattr(config, "point_path") or hasattr(config, "init_points_num")):
        loaded_iter, config, aabb = config, aabb, (reference_tail[0] if reference_tail else None)
        model = reference_tail[2] if len(reference_tail) > 2 else None
        if loaded_iter:
            model.load_from_state_dict(model.get_state_dict_from_ckpt(config.ckpt, config.device))
            return None
        if not getattr(config, "point_path", None) and str(getattr(config, "dataset_name", "")).lower() == "colmap":
            return init_ply(config.datadir, aabb, "colmap", int(getattr(config, "init_points_num", 100_000)))
        return get_pcd(config, aabb)
    path = getattr(config, "point_path", None)
    if not path and dataset is not None and hasattr(dataset, "initial_point_cloud"):
        xyz, rgb = dataset.initial_point_cloud()
        if xyz is not None and len(xyz) > 0:
            pcd = BasicPointCloud(points=np.asarray(xyz, dtype=np.float32), colors=np.asarray(rgb, dtype=np.float32),
                                  normals=np.zeros((len(xyz), 3), dtype=np.float32))
            return _cap_points(pcd, int(getattr(config, "max_init_points", -1)))
    if path:
        pcd = fetchLas(path) if path.endswith(".las") else fetchPly(path)
    else:
        assert aabb is not None, "an AABB is needed to draw the initial random cloud"
        rng = np.random.default_rng(int(getattr(config, "random_seed", 0)))
        lb, ub = np.asarray(aabb[0], dtype=np.float32), np.asarray(aabb[1], dtype=np.float32)
        n = int(getattr(config, "init_points_num", 100_000))
        xyz = rng.random((n, 3), dtype=np.float32) * (ub - lb) + lb
        if not getattr(config, "init_points_volume", False):
            xyz[:, 2] = lb[2]
        pcd = BasicPointCloud(points=xyz, colors=rng.random((n, 3), dtype=np.float32), normals=np.zeros_like(xyz))
    return _cap_points(pcd, int(getattr(config, "max_init_points", -1)))


def _cap_points(pcd: BasicPointCloud, limit: int) -> BasicPointCloud:
    if limit > 0 and len(pcd.points) > limit:
        keep = np.random.default_rng(0).choice(len(pcd.points), limit, replace=False)
        pcd = BasicPointCloud(pcd.points[keep], pcd.colors[keep], pcd.normals[keep])
    return pcd
