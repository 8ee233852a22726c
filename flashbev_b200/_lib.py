"""ctypes binding of libfbev.so, the C ABI declared in include/fbev.h.

There is no fallback: if the library cannot be loaded the import of the operator
fails with the reason, and nothing is computed on the CPU instead.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

F32, BF16, F16 = 0, 1, 2
DEPTH_GAUSSIAN, DEPTH_LAPLACE, DEPTH_CATEGORICAL, DEPTH_CATEGORICAL_LOGITS = 0, 1, 2, 3
ABI_VERSION = 2
POOL_MEAN, POOL_SUM = 0, 1
BWD_FEATS, BWD_DEPTH, BWD_LEGACY_DEPTH, BWD_DETERMINISTIC = 1, 2, 4, 8
DEV_BAD_FEATURE_SIZE = 1
WORKSPACE_BYTES = 16
STATIC_SCRATCH_BYTES = 16 << 20
SORT_BUDGET_BYTES = 256 << 20
ERR_SCRATCH = 8
ERR_STATIC_LIMIT = 11

# every symbol include/fbev.h declares (the operator) ...
EXPORTS = (
    "fbev_forward", "fbev_forward_to_host", "fbev_forward_peers", "fbev_forward_multicast", "fbev_backward", "fbev_backward_scratch_bytes", "fbev_backward_min_scratch_bytes", "fbev_saved_state_bytes", "fbev_backward_static_scratch",
    "fbev_debug_indices",
    "fbev_flash_bevpool", "fbev_flash_bevpool_grad", "fbev_projection_matrices", "fbev_pillar_pool",
    "fbev_strerror", "fbev_version", "fbev_source_hash",
)
# ... and include/fbev_debug.h (experiment and test helpers)
DEBUG_EXPORTS = ("fbev_set_tuning", "fbev_set_experiment", "fbev_probe_read")
EXP_PREFETCH, EXP_GROUP_CULL, EXP_DRAW, EXP_SHARED_GATHER_CEILING = 1, 2, 4, 8


class FbevProblem(ctypes.Structure):
    """Mirror of ``struct FbevProblem`` (include/fbev.h)."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("B", ctypes.c_int32), ("N", ctypes.c_int32), ("H", ctypes.c_int32), ("W", ctypes.c_int32),
        ("C", ctypes.c_int32),
        ("D", ctypes.c_int32),
        ("X", ctypes.c_int32), ("Y", ctypes.c_int32), ("Z", ctypes.c_int32),
        ("proj_stride", ctypes.c_int32),
        ("mode", ctypes.c_int32),
        ("pool", ctypes.c_int32),
        ("epsilon", ctypes.c_float),
        ("threshold", ctypes.c_float),
        ("depth_d0", ctypes.c_float), ("depth_delta", ctypes.c_float),
        ("y_begin", ctypes.c_int32), ("y_end", ctypes.c_int32),
        ("voxel_size", ctypes.c_float * 3),
        ("voxel_min", ctypes.c_float * 3),
        ("compact_rows", ctypes.c_int32),
        ("image_feats", ctypes.c_void_p),
        ("depth", ctypes.c_void_p),
        ("projection", ctypes.c_void_p),
        ("feature_size", ctypes.c_void_p),
        ("image_size", ctypes.c_void_p),
        ("roi_range", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("saved_state", ctypes.c_void_p),
        ("saved_state_bytes", ctypes.c_uint64),
        ("depth_stats", ctypes.c_void_p),
    ]


class FbevError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: {strerror(status)} (status {status})")
        self.status = status


_lib = None


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Loads libfbev.so, compiling it first when it is missing or was built from other sources than the ones
    beside it (compared by content hash) and nvcc is available.  A library whose embedded hash does not match
    the sources is refused: kernels of another version never run silently."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if _build.is_stale():
        if not build_if_missing:
            raise ImportError(f"{path} is missing or stale; build it with `python -m flashbev_b200.build`")
        _build.build()
    lib = ctypes.CDLL(path)
    lib.fbev_source_hash.restype = ctypes.c_char_p
    built_from = lib.fbev_source_hash().decode()
    if built_from != _build.source_hash():
        raise ImportError(f"{path} was built from other sources (hash {built_from[:12]}...) than the ones in "
                          f"{_build.CSRC}; rebuild it with `python -m flashbev_b200.build --force`")
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.fbev_forward.argtypes = [ctypes.POINTER(FbevProblem), vp, vp, vp]
    lib.fbev_forward.restype = i32
    lib.fbev_forward_to_host.argtypes = [ctypes.POINTER(FbevProblem), vp, vp, i32, vp]
    lib.fbev_forward_to_host.restype = i32
    lib.fbev_forward_peers.argtypes = [ctypes.POINTER(FbevProblem), vp, ctypes.POINTER(vp), i32, vp, vp]
    lib.fbev_forward_peers.restype = i32
    lib.fbev_forward_multicast.argtypes = [ctypes.POINTER(FbevProblem), vp, vp, vp, vp]
    lib.fbev_forward_multicast.restype = i32
    lib.fbev_backward_scratch_bytes.argtypes = [ctypes.POINTER(FbevProblem), i32]
    lib.fbev_backward_scratch_bytes.restype = ctypes.c_size_t
    lib.fbev_saved_state_bytes.argtypes = [ctypes.POINTER(FbevProblem)]
    lib.fbev_saved_state_bytes.restype = ctypes.c_size_t
    lib.fbev_backward_min_scratch_bytes.argtypes = [ctypes.POINTER(FbevProblem), i32]
    lib.fbev_backward_min_scratch_bytes.restype = ctypes.c_size_t
    lib.fbev_backward.argtypes = [ctypes.POINTER(FbevProblem), vp, vp, vp, vp, ctypes.c_size_t, i32, vp]
    lib.fbev_backward.restype = i32
    lib.fbev_backward_static_scratch.argtypes = [ctypes.POINTER(FbevProblem), vp, vp, vp, i32, vp]
    lib.fbev_backward_static_scratch.restype = i32
    lib.fbev_debug_indices.argtypes = [ctypes.POINTER(FbevProblem), vp, vp, vp, vp, vp, vp]
    lib.fbev_debug_indices.restype = i32
    lib.fbev_flash_bevpool.argtypes = [i32] * 11 + [f32, f32] + [vp] * 5 + [i32] * 3 + [f32] * 6 + [vp, vp]
    lib.fbev_flash_bevpool.restype = i32
    lib.fbev_flash_bevpool_grad.argtypes = [i32] * 7 + [f32, f32] + [vp] * 7 + [i32] * 3 + [vp, vp, i32, i32, vp]
    lib.fbev_flash_bevpool_grad.restype = i32
    lib.fbev_projection_matrices.argtypes = [vp] * 5 + [i32, vp]
    lib.fbev_projection_matrices.restype = i32
    lib.fbev_pillar_pool.argtypes = [i32, i32] + [vp] * 9 + [i32] * 4 + [f32, i32, vp, vp]
    lib.fbev_pillar_pool.restype = i32
    lib.fbev_set_tuning.argtypes = [i32] * 5
    lib.fbev_set_tuning.restype = None
    lib.fbev_set_experiment.argtypes = [i32]
    lib.fbev_set_experiment.restype = None
    lib.fbev_probe_read.argtypes = [vp, ctypes.c_size_t, i32, vp, vp]
    lib.fbev_probe_read.restype = i32
    lib.fbev_strerror.argtypes = [i32]
    lib.fbev_strerror.restype = ctypes.c_char_p
    lib.fbev_version.restype = i32
    if lib.fbev_version() != ABI_VERSION:
        raise ImportError(f"{path}: ABI version {lib.fbev_version()} != {ABI_VERSION}")
    _lib = lib
    return lib


def strerror(status: int) -> str:
    return load().fbev_strerror(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != 0:
        raise FbevError(status, what)
