"""Builds the native library in-tree: ``edmir_b200/libedm_b200.so``.

The kernels use tcgen05 / TMEM / TMA and therefore compile for sm_100a only.  nvcc
cross-compiles without a GPU, so this runs on any host with the CUDA toolkit.

    python -m edmir_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libedm_b200.so")
SOURCES = ["edm_api.cu", "selector.cpp"]
HEADERS = ["ptx.cuh", "tp_gemm.cuh", "moe.cuh", "ar_oneshot.cuh", "decode_gemm.cuh", os.path.join("..", "..", "include", "edm_b200.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the native library cannot be built")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


CHECKED_LIB_PATH = os.path.join(PKG_DIR, "libedm_b200_checked.so")


def build_checked(verbose: bool = False) -> str:
    """Compile the checking variant (``-DEDM_DEBUG_BOUNDS``): every global address the kernel
    computes is validated against the ranges the launch may touch and violations are reported
    through the status words instead of faulting.  Select it with ``EDM_LIB_PATH``."""
    return build(force=True, verbose=verbose, out=CHECKED_LIB_PATH, defines=("EDM_DEBUG_BOUNDS",))


def build(force: bool = False, verbose: bool = False, out: str = LIB_PATH, defines: tuple = ()) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if out == LIB_PATH and not force and not _stale():
        return LIB_PATH
    tmp = f"{out}.{os.getpid()}.tmp"   # a reader never sees a half-written library
    cmd = [
        _nvcc(), "-shared", "-Xcompiler", "-fPIC", "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-o", tmp,
    ] + [f"-D{d}" for d in defines] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError(f"nvcc failed building {os.path.basename(out)}")
    os.replace(tmp, out)
    return out


if __name__ == "__main__":
    if "--checked" in sys.argv:
        print(build_checked(verbose="--verbose" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
