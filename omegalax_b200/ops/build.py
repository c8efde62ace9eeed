"""In-tree build of the sm_100a CUDA library.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``
into an object and the objects are linked into ``omegalax_b200/ops/libomegalax_b200.so``.
The library exposes plain ``extern "C"`` launchers that take raw device pointers and a
stream, so it has no dependency on libtorch and builds in seconds; Python binds it with
ctypes (see ``lib.py``).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = HERE / "libomegalax_b200.so"
DEBUG_LIB = HERE / "libomegalax_b200_debug.so"
# debug build: GEMM epilogues check every store against the output's extent and record status 8;
# bounded waits give up after ~0.2 s so a protocol error surfaces quickly
DEBUG_FLAGS = ["-DOB_DEBUG_BOUNDS", "-DOB_WAIT_CYCLES=400000000ll"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def sources():
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared library (``debug``: the variant with
    in-kernel store checks and short wait budgets, ``libomegalax_b200_debug.so``)."""
    srcs = sources()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    out_lib = DEBUG_LIB if debug else LIB
    build_dir = BUILD / "debug" if debug else BUILD
    extra = DEBUG_FLAGS if debug else []
    stamp = build_dir / "stamp.txt"
    want = _digest(srcs + headers) + ("-debug" if debug else "")
    if not force and out_lib.exists() and stamp.exists() and stamp.read_text() == want:
        return out_lib
    build_dir.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: Path) -> Path:
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [nvcc, "-shared", "-o", str(out_lib), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(want)
    return out_lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug="--debug" in sys.argv))
