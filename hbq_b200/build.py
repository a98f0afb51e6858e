"""Build step: compile the CUDA sources under ``csrc/`` into ``lib/libhbq_b200.so``.

The library targets sm_100a only and depends on nothing but the CUDA runtime, so it
cross-compiles on a machine without a GPU::

    python -m hbq_b200.build
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libhbq_b200.so")
SOURCES = ["api.cu", "quantize.cu", "quantize_lut.cu", "quantize_tab.cu", "quantize_extra.cu", "gemm_simt.cu", "gemm_tc.cu", "gemm_packed.cu", "gemm_static.cu"]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "quantize_dev.cuh"), os.path.join(CSRC, "vcache_dev.cuh"), os.path.join(CSRC, "quantize_tab.cuh"), os.path.join(CSRC, "tc_dev.cuh"), os.path.join(HERE, "..", "include", "hbq_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "--threads", "4"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; it is needed to build libhbq_b200.so")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile if the shared object is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, *[os.path.join(CSRC, s) for s in SOURCES]]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    env = dict(os.environ)
    # nvcc's host compiler: the image exports a CC wrapper that is not a full gcc install
    env.pop("CC", None)
    env.pop("CXX", None)
    subprocess.check_call(cmd, env=env)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
