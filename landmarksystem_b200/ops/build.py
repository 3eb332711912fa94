"""In-tree build of the sm_100a CUDA libraries.

Every ``csrc/*.cu`` is compiled by ``nvcc -gencode arch=compute_100a,code=sm_100a`` into an
object file and linked into ``_lib/liblmb200.so`` beside this file.  The library exposes a plain
C ABI (raw device pointers + ``cudaStream_t``) that :mod:`landmarksystem_b200.ops.native`
binds with ``ctypes``; nothing depends on torch's C++ headers, so a full rebuild takes seconds
and cross-compiles on a machine without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "_lib"
LIB_NAME = "liblmb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


# Approximate division / square root / transcendental code (``--use_fast_math``) only where the arithmetic is a small
# part of a bandwidth- or tensor-core-bound kernel whose tests compare against bf16-level tolerances.  Everything else -
# the optimisers, the compositor, the samplers, the losses - is compiled with IEEE arithmetic.
# ``lazy_adam`` replays up to 192 skipped Adam steps per texel in registers (a division and a square root per step and
# channel): with IEEE division the deferred update is four times slower than the dense sweep it replaces.
FAST_MATH_UNITS = {"fused_mlp", "fused_mlp_bwd", "gs_raster", "hashgrid", "gs_aux", "lazy_adam"}


def _flags_for(src: Path):
    return NVCC_FLAGS + (["--use_fast_math"] if src.stem in FAST_MATH_UNITS else [])


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _digest(path: Path, headers) -> str:
    h = hashlib.sha1()
    h.update(path.read_bytes())
    for hdr in headers:
        h.update(hdr.read_bytes())
    h.update(" ".join(_flags_for(path)).encode())
    return h.hexdigest()


def _compile_one(src: Path, headers, verbose: bool) -> Path:
    OUT.mkdir(exist_ok=True)
    obj = OUT / (src.stem + ".o")
    stamp = OUT / (src.stem + ".sha1")
    want = _digest(src, headers)
    if obj.exists() and stamp.exists() and stamp.read_text() == want:
        return obj
    cmd = [_nvcc(), *_flags_for(src), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (OUT / (src.stem + ".ptxas.log")).write_text(res.stderr)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"nvcc failed for {src.name}")
    if verbose:
        print(f"[lmb200 build] compiled {src.name}")
    stamp.write_text(want)
    return obj


def library_path() -> Path:
    return OUT / LIB_NAME


def build_all(verbose: bool = False, force: bool = False) -> Path:
    """Compile every kernel source and link the shared library; returns its path."""
    if force and OUT.exists():
        for f in OUT.glob("*.sha1"):
            f.unlink()
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    if not sources:
        raise RuntimeError("no CUDA sources found")
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, headers, verbose), sources))
    lib = library_path()
    newest = max(o.stat().st_mtime for o in objs)
    if (not lib.exists()) or lib.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(lib), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
        if verbose:
            print(f"[lmb200 build] linked {lib}")
    return lib


def resource_digest() -> str:
    """Markdown table of what ptxas reported for every kernel of the last build: registers, shared memory, stack frame
    and spill bytes (the compiler's own ``-Xptxas -v`` lines, nothing is disassembled)."""
    import re

    rows = []
    for log in sorted(OUT.glob("*.ptxas.log")):
        name = None
        stack = spill_st = spill_ld = 0
        for line in log.read_text().splitlines():
            m = re.search(r"Compiling entry function '([^']+)'", line)
            if m:
                name = m.group(1)
                continue
            m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
            if m:
                stack, spill_st, spill_ld = (int(v) for v in m.groups())
                continue
            m = re.search(r"Used (\d+) registers(.*)", line)
            if m and name:
                smem = re.search(r"(\d+) bytes smem", m.group(2))
                rows.append((log.name.replace(".ptxas.log", ".cu"), name, int(m.group(1)), int(smem.group(1)) if smem else 0,
                             stack, spill_st, spill_ld))
                name = None
    try:
        res = subprocess.run(["c++filt"], input="\n".join(r[1] for r in rows), capture_output=True, text=True)
        pretty = res.stdout.splitlines() if res.returncode == 0 else [r[1] for r in rows]
    except OSError:
        pretty = [r[1] for r in rows]
    out = ["| file | kernel | registers | static smem (B) | stack (B) | spill st / ld (B) |", "|---|---|---|---|---|---|"]
    for (src, _, regs, smem, stack, st, ld), nice in zip(rows, pretty):
        nice = re.sub(r"\(.*", "", nice).replace("lmb::", "").replace("void ", "")
        out.append(f"| {src} | `{nice}` | {regs} | {smem} | {stack} | {st} / {ld} |")
    return "\n".join(out)


if __name__ == "__main__":
    build_all(verbose=True, force="--force" in sys.argv)
    print(library_path())
    if "--digest" in sys.argv:
        print(resource_digest())
