"""Builds libfbev.so (sm_100a only) in-tree with nvcc.  No torch headers are involved.

    python -m flashbev_b200.build [--force]

The shared library is written next to this file so that it travels with the source
tree; it is the only native artefact of the package.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libfbev.so")
SOURCES = ["fbev_kernels.cu"]
HEADERS = sorted(os.path.join(CSRC, h) for h in os.listdir(CSRC) if h.endswith(".cuh")) + \
          [os.path.join(INCLUDE, "fbev.h"), os.path.join(INCLUDE, "fbev_debug.h")]
HASH_PATH = LIB_PATH + ".srchash"  # hash of the sources the library beside it was built from

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


def source_hash() -> str:
    """SHA-256 over the library's sources and the compiler flags, in a fixed order."""
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for path in [os.path.join(CSRC, s) for s in SOURCES] + HEADERS:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def is_stale() -> bool:
    """True when the library is missing or was built from other sources than the ones present (compared by
    content, not by time stamp: a copied tree keeps its library and must not rebuild it)."""
    if not (os.path.exists(LIB_PATH) and os.path.exists(HASH_PATH)):
        return True
    with open(HASH_PATH) as fh:
        return fh.read().strip() != source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    digest = source_hash()
    tmp = LIB_PATH + f".tmp{os.getpid()}"
    cmd = [find_nvcc()] + NVCC_FLAGS + [f'-DFBEV_SOURCE_HASH="{digest}"', "-I", INCLUDE, "-I", CSRC, "-o", tmp] + \
          [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError("nvcc failed building libfbev.so")
    os.replace(tmp, LIB_PATH)  # atomic: a process loading the library meanwhile sees the old or the new file
    with open(HASH_PATH, "w") as fh:
        fh.write(digest + "\n")
    with open(os.path.join(PKG_DIR, "libfbev.ptxas.txt"), "w") as fh:  # register / spill report of the build
        fh.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
