"""Builds libb200q.so (CUDA kernels + C ABI) in-tree for sm_100a with nvcc.

Every source is compiled to an object of its own (in parallel, and only when it or a header changed), then
linked; objects live in `chadslab_b200/_obj/`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libb200q.so")
SOURCES = ["api.cu", "simt.cu", "gemv_mma.cu", "gemv_push.cu", "gemv_gated.cu", "gemv_batch.cu", "moe.cu", "tc.cu", "glue.cu", "attn_mma.cu", "comm.cu", "ep.cu", "quant.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libb200q.so cannot be built")
    return exe


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [
        os.path.join(HERE, "..", "include", "b200q.h")]


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def needs_build() -> bool:
    return _stale(LIB, [os.path.join(CSRC, s) for s in SOURCES] + _headers())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc, hdrs = _nvcc(), _headers()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str):
        obj = os.path.join(OBJ, src[:-3] + ".o")
        path = os.path.join(CSRC, src)
        if not (force or verbose) and not _stale(obj, [path] + hdrs):
            return obj, ""
        r = subprocess.run([nvcc, *NVCC_FLAGS, *extra, "-c", path, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n" + r.stdout + r.stderr)
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    if verbose:
        sys.stderr.write("".join(err for _, err in results))
    r = subprocess.run([nvcc, "-shared", "-o", LIB] + [o for o, _ in results] + ["-lcuda"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
