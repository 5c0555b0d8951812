"""Builds libl2j_b200.so (the CUDA kernels and the C ABI) for sm_100a with nvcc.

The library is built in-tree next to this file so that it travels with the source tree; it is
never installed into site-packages.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libl2j_b200.so")
SOURCES = ["l2j_kernels.cu", "l2j_fused.cu", "l2j_sampler.cu", "l2j_prefill.cu", "l2j_api.cu", "l2j_noalloc.cu"]
HEADERS = ["l2j_device.cuh", "l2j_internal.h", os.path.join("..", "..", "include", "l2j_b200.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put /usr/local/cuda/bin on PATH)")


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None) -> str:
    """Compiles every CUDA source for sm_100a into one shared object and returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-lineinfo", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2",
        "-ccbin", "g++",
        "-Xptxas", "-v" if verbose else "-O3",
        "-o", LIB_PATH,
    ]
    cmd += list(extra_flags or [])
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
