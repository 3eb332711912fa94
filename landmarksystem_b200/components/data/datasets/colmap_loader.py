"""Readers (and writers, used by tests and converters) for COLMAP sparse models: ``cameras``, ``images`` and
``points3D`` in the binary and the text format (reference role: landmark/nerf_components/data/datasets/
dataloader/utils/colmap_loader.py).  Only ``numpy`` and ``struct`` are needed."""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass
from typing import BinaryIO, Dict, Tuple

import numpy as np

# model id -> (name, number of parameters), as defined by COLMAP's camera_models
CAMERA_MODELS = {0: ("SIMPLE_PINHOLE", 3), 1: ("PINHOLE", 4), 2: ("SIMPLE_RADIAL", 4), 3: ("RADIAL", 5), 4: ("OPENCV", 8),
                 5: ("OPENCV_FISHEYE", 8), 6: ("FULL_OPENCV", 12), 7: ("FOV", 5), 8: ("SIMPLE_RADIAL_FISHEYE", 4),
                 9: ("RADIAL_FISHEYE", 5), 10: ("THIN_PRISM_FISHEYE", 12)}
MODEL_IDS = {name: (mid, n) for mid, (name, n) in CAMERA_MODELS.items()}


@dataclass
class ColmapCamera:
    id: int
    model: str
    width: int
    height: int
    params: np.ndarray

    def focal(self) -> Tuple[float, float]:
        if self.model in ("SIMPLE_PINHOLE", "SIMPLE_RADIAL", "RADIAL", "SIMPLE_RADIAL_FISHEYE", "RADIAL_FISHEYE"):
            return float(self.params[0]), float(self.params[0])
        return float(self.params[0]), float(self.params[1])


@dataclass
class ColmapImage:
    id: int
    qvec: np.ndarray          # world-to-camera rotation as (w, x, y, z)
    tvec: np.ndarray          # world-to-camera translation
    camera_id: int
    name: str
    xys: np.ndarray
    point3D_ids: np.ndarray

    def rotation(self) -> np.ndarray:
        return qvec2rotmat(self.qvec)


def qvec2rotmat(q: np.ndarray) -> np.ndarray:
    w, x, y, z = [float(v) for v in q]
    return np.array([[1 - 2 * y * y - 2 * z * z, 2 * x * y - 2 * w * z, 2 * z * x + 2 * w * y],
                     [2 * x * y + 2 * w * z, 1 - 2 * x * x - 2 * z * z, 2 * y * z - 2 * w * x],
                     [2 * z * x - 2 * w * y, 2 * y * z + 2 * w * x, 1 - 2 * x * x - 2 * y * y]])


def rotmat2qvec(R: np.ndarray) -> np.ndarray:
    """Inverse of :func:`qvec2rotmat` (Shepperd's method, w >= 0)."""
    R = np.asarray(R, dtype=np.float64)
    t = np.trace(R)
    if t > 0:
        s = np.sqrt(t + 1.0) * 2
        q = np.array([0.25 * s, (R[2, 1] - R[1, 2]) / s, (R[0, 2] - R[2, 0]) / s, (R[1, 0] - R[0, 1]) / s])
    else:
        i = int(np.argmax(np.diag(R)))
        j, k = (i + 1) % 3, (i + 2) % 3
        s = np.sqrt(R[i, i] - R[j, j] - R[k, k] + 1.0) * 2
        q = np.zeros(4)
        q[0] = (R[k, j] - R[j, k]) / s
        q[1 + i] = 0.25 * s
        q[1 + j] = (R[j, i] + R[i, j]) / s
        q[1 + k] = (R[k, i] + R[i, k]) / s
    return -q if q[0] < 0 else q


def _unpack(fh: BinaryIO, fmt: str):
    return struct.unpack("<" + fmt, fh.read(struct.calcsize("<" + fmt)))


# -- binary ---------------------------------------------------------------------------------------------
def read_cameras_binary(path: str) -> Dict[int, ColmapCamera]:
    out = {}
    with open(path, "rb") as fh:
        (n,) = _unpack(fh, "Q")
        for _ in range(n):
            cam_id, model_id, width, height = _unpack(fh, "iiQQ")
            name, n_params = CAMERA_MODELS[model_id]
            out[cam_id] = ColmapCamera(cam_id, name, int(width), int(height), np.array(_unpack(fh, "d" * n_params)))
    return out


def read_images_binary(path: str) -> Dict[int, ColmapImage]:
    out = {}
    with open(path, "rb") as fh:
        (n,) = _unpack(fh, "Q")
        for _ in range(n):
            vals = _unpack(fh, "idddddddi")
            image_id, qvec, tvec, camera_id = vals[0], np.array(vals[1:5]), np.array(vals[5:8]), vals[8]
            name = b""
            while True:
                ch = fh.read(1)
                if ch in (b"\x00", b""):
                    break
                name += ch
            (n_pts,) = _unpack(fh, "Q")
            raw = np.frombuffer(fh.read(24 * n_pts), dtype=np.dtype([("x", "<f8"), ("y", "<f8"), ("id", "<i8")]))
            out[image_id] = ColmapImage(image_id, qvec, tvec, camera_id, name.decode("utf-8"),
                                        np.stack((raw["x"], raw["y"]), -1) if n_pts else np.zeros((0, 2)),
                                        raw["id"].copy() if n_pts else np.zeros((0,), np.int64))
    return out


def read_points3D_binary(path: str):
    """Returns ``(xyz [N,3] float64, rgb [N,3] uint8, error [N])``; track lists are skipped."""
    with open(path, "rb") as fh:
        (n,) = _unpack(fh, "Q")
        xyz, rgb, err = np.empty((n, 3)), np.empty((n, 3), np.uint8), np.empty(n)
        for k in range(n):
            vals = _unpack(fh, "QdddBBBd")
            xyz[k], rgb[k], err[k] = vals[1:4], vals[4:7], vals[7]
            (track,) = _unpack(fh, "Q")
            fh.seek(8 * track, os.SEEK_CUR)
    return xyz, rgb, err


# -- text -----------------------------------------------------------------------------------------------
def _data_lines(path: str):
    with open(path, encoding="utf-8") as fh:
        for line in fh:
            line = line.strip()
            if line and not line.startswith("#"):
                yield line


def read_cameras_text(path: str) -> Dict[int, ColmapCamera]:
    out = {}
    for line in _data_lines(path):
        tok = line.split()
        out[int(tok[0])] = ColmapCamera(int(tok[0]), tok[1], int(tok[2]), int(tok[3]), np.array([float(v) for v in tok[4:]]))
    return out


def read_images_text(path: str) -> Dict[int, ColmapImage]:
    out = {}
    with open(path, encoding="utf-8") as fh:
        lines = [l.rstrip("\n") for l in fh if not l.startswith("#")]
    k = 0
    while k < len(lines):
        if not lines[k].strip():
            k += 1
            continue
        tok = lines[k].split()
        pts = lines[k + 1].split() if k + 1 < len(lines) else []
        xys = np.array([[float(pts[i]), float(pts[i + 1])] for i in range(0, len(pts) - 2, 3)]).reshape(-1, 2)
        ids = np.array([int(pts[i + 2]) for i in range(0, len(pts) - 2, 3)], dtype=np.int64)
        out[int(tok[0])] = ColmapImage(int(tok[0]), np.array([float(v) for v in tok[1:5]]), np.array([float(v) for v in tok[5:8]]),
                                       int(tok[8]), tok[9], xys, ids)
        k += 2
    return out


def read_points3D_text(path: str):
    rows = [line.split() for line in _data_lines(path)]
    xyz = np.array([[float(v) for v in r[1:4]] for r in rows]).reshape(-1, 3)
    rgb = np.array([[int(v) for v in r[4:7]] for r in rows], dtype=np.uint8).reshape(-1, 3)
    err = np.array([float(r[7]) for r in rows])
    return xyz, rgb, err


def read_model(sparse_dir: str):
    """``(cameras, images, (xyz, rgb, err))`` from a ``sparse/0`` style directory, binary preferred over text."""
    def pick(stem):
        for ext, binary in ((".bin", True), (".txt", False)):
            path = os.path.join(sparse_dir, stem + ext)
            if os.path.exists(path):
                return path, binary
        raise FileNotFoundError(f"no {stem}.bin / {stem}.txt under {sparse_dir}")

    cpath, cbin = pick("cameras")
    ipath, ibin = pick("images")
    cameras = read_cameras_binary(cpath) if cbin else read_cameras_text(cpath)
    images = read_images_binary(ipath) if ibin else read_images_text(ipath)
    try:
        ppath, pbin = pick("points3D")
        points = read_points3D_binary(ppath) if pbin else read_points3D_text(ppath)
    except FileNotFoundError:
        points = (np.zeros((0, 3)), np.zeros((0, 3), np.uint8), np.zeros(0))
    return cameras, images, points


# -- writers --------------------------------------------------------------------------------------------
def write_model_binary(sparse_dir: str, cameras: Dict[int, ColmapCamera], images: Dict[int, ColmapImage], points) -> None:
    os.makedirs(sparse_dir, exist_ok=True)
    with open(os.path.join(sparse_dir, "cameras.bin"), "wb") as fh:
        fh.write(struct.pack("<Q", len(cameras)))
        for cam in cameras.values():
            fh.write(struct.pack("<iiQQ", cam.id, MODEL_IDS[cam.model][0], cam.width, cam.height))
            fh.write(struct.pack("<" + "d" * len(cam.params), *[float(v) for v in cam.params]))
    with open(os.path.join(sparse_dir, "images.bin"), "wb") as fh:
        fh.write(struct.pack("<Q", len(images)))
        for im in images.values():
            fh.write(struct.pack("<idddddddi", im.id, *[float(v) for v in im.qvec], *[float(v) for v in im.tvec], im.camera_id))
            fh.write(im.name.encode("utf-8") + b"\x00")
            fh.write(struct.pack("<Q", len(im.point3D_ids)))
            for (x, y), pid in zip(im.xys, im.point3D_ids):
                fh.write(struct.pack("<ddq", float(x), float(y), int(pid)))
    xyz, rgb, err = points
    with open(os.path.join(sparse_dir, "points3D.bin"), "wb") as fh:
        fh.write(struct.pack("<Q", len(xyz)))
        for k in range(len(xyz)):
            fh.write(struct.pack("<QdddBBBd", k + 1, *[float(v) for v in xyz[k]], *[int(v) for v in rgb[k]], float(err[k])))
            fh.write(struct.pack("<Q", 0))


def write_model_text(sparse_dir: str, cameras, images, points) -> None:
    os.makedirs(sparse_dir, exist_ok=True)
    with open(os.path.join(sparse_dir, "cameras.txt"), "w", encoding="utf-8") as fh:
        fh.write("# Camera list with one line of data per camera:\n#   CAMERA_ID, MODEL, WIDTH, HEIGHT, PARAMS[]\n")
        for cam in cameras.values():
            fh.write(f"{cam.id} {cam.model} {cam.width} {cam.height} " + " ".join(repr(float(v)) for v in cam.params) + "\n")
    with open(os.path.join(sparse_dir, "images.txt"), "w", encoding="utf-8") as fh:
        fh.write("# IMAGE_ID, QW, QX, QY, QZ, TX, TY, TZ, CAMERA_ID, NAME\n#   POINTS2D[] as (X, Y, POINT3D_ID)\n")
        for im in images.values():
            fh.write(f"{im.id} " + " ".join(repr(float(v)) for v in list(im.qvec) + list(im.tvec)) + f" {im.camera_id} {im.name}\n")
            fh.write(" ".join(f"{float(x)!r} {float(y)!r} {int(p)}" for (x, y), p in zip(im.xys, im.point3D_ids)) + "\n")
    xyz, rgb, err = points
    with open(os.path.join(sparse_dir, "points3D.txt"), "w", encoding="utf-8") as fh:
        fh.write("# POINT3D_ID, X, Y, Z, R, G, B, ERROR, TRACK[]\n")
        for k in range(len(xyz)):
            fh.write(f"{k + 1} " + " ".join(repr(float(v)) for v in xyz[k]) + " " + " ".join(str(int(v)) for v in rgb[k])
                     + f" {float(err[k])!r}\n")


# -- dense-reconstruction arrays and the names the 3DGS code base uses for the readers -----------------------------
def read_colmap_bin_array(path: str) -> np.ndarray:
    """A COLMAP dense array (depth / normal map): text header ``width&height&channels&`` followed by float32 values in
    column-major order; returns ``[height, width]`` or ``[height, width, channels]``."""
    with open(path, "rb") as fh:
        header = b""
        while header.count(b"&") < 3:
            byte = fh.read(1)
            assert byte, f"{path}: truncated header"
            header += byte
        width, height, channels = (int(v) for v in header.split(b"&")[:3])
        data = np.frombuffer(fh.read(), dtype=np.float32, count=width * height * channels)
    return np.transpose(data.reshape((width, height, channels), order="F"), (1, 0, 2)).squeeze()


def write_colmap_bin_array(path: str, array: np.ndarray) -> None:
    """Inverse of :func:`read_colmap_bin_array`."""
    a = np.asarray(array, dtype=np.float32)
    a = a[..., None] if a.ndim == 2 else a
    height, width, channels = a.shape
    with open(path, "wb") as fh:
        fh.write(f"{width}&{height}&{channels}&".encode("ascii"))
        fh.write(np.transpose(a, (1, 0, 2)).reshape(-1, order="F").tobytes())


def read_next_bytes(fid: BinaryIO, num_bytes: int, format_char_sequence: str, endian_character: str = "<"):
    """Read and unpack the next ``num_bytes`` of a binary model file."""
    return struct.unpack(endian_character + format_char_sequence, fid.read(num_bytes))


Camera = ColmapCamera                                   # record names of the reference's loader
Image = ColmapImage
read_extrinsics_binary, read_extrinsics_text = read_images_binary, read_images_text
read_intrinsics_binary, read_intrinsics_text = read_cameras_binary, read_cameras_text
