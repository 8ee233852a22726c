"""Builds libfbev.so (sm_100a only) in-tree with nvcc.  No torch headers are involved.

    python -m flashbev_b200.build [--force]

The shared library is written next to this file so that it travels with the source
tree; it is the only native artefact of the package.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libfbev.so")
SOURCES = ["fbev_kernels.cu"]
HEADERS = [os.path.join(CSRC, h) for h in ("fbev_device.cuh", "fbev_lists.cuh", "fbev_forward.cuh", "fbev_backward.cuh",
                                            "fbev_sort.cuh", "fbev_misc.cuh")] + [os.path.join(INCLUDE, "fbev.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def find_nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: libfbev.so cannot be built (CUDA 12.8+ with sm_100a support is required)")
    return cand


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [find_nvcc()] + NVCC_FLAGS + ["-I", INCLUDE, "-I", CSRC, "-o", LIB_PATH] + \
          [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libfbev.so")
    with open(os.path.join(PKG_DIR, "libfbev.ptxas.txt"), "w") as fh:  # register / spill report of the build
        fh.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
