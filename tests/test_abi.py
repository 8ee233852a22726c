"""CPU checks of the C ABI: libfbev.so loads, exports every symbol include/fbev.h declares, and
its host-side validation returns status codes (no kernel is launched here)."""
import ctypes
import glob
import os
import re

import pytest
import torch

from flashbev_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    """Every function declared in include/*.h (fbev.h: the operator; fbev_debug.h: experiment helpers)."""
    names = set()
    for path in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        text = re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)
        names |= set(re.findall(r"\b(fbev_[a-z_0-9]+)\s*\(", text))
    return sorted(names)


def test_header_and_binding_list_the_same_functions():
    assert header_functions() == sorted(_lib.EXPORTS + _lib.DEBUG_EXPORTS)


def test_library_builds_and_exports_every_symbol():
    build.build()
    lib = ctypes.CDLL(build.LIB_PATH)
    for name in header_functions():
        assert hasattr(lib, name), name
    assert _lib.load().fbev_version() == _lib.ABI_VERSION == 2


def test_struct_layout_matches_the_header():
    # uint32 + 20 int32/float words + 6 floats + compact_rows = 28 words, then 8 pointers, saved_state and its
    # 64-bit size, depth_stats (LP64)
    assert ctypes.sizeof(_lib.FbevProblem) == 4 * 28 + 8 * 11
    assert _lib.FbevProblem.compact_rows.offset == 108 and _lib.FbevProblem.image_feats.offset == 112 and _lib.FbevProblem.workspace.offset == 168
    assert _lib.FbevProblem.saved_state.offset == 176 and _lib.FbevProblem.depth_stats.offset == 192


def _problem():
    p = _lib.FbevProblem()
    p.struct_size = ctypes.sizeof(_lib.FbevProblem)
    p.dtype = _lib.F32
    p.out_dtype = _lib.F32
    p.B, p.N, p.H, p.W, p.C, p.D = 1, 2, 4, 4, 8, 2
    p.X, p.Y, p.Z = 8, 8, 2
    p.proj_stride = 12
    p.mode, p.pool = _lib.DEPTH_LAPLACE, _lib.POOL_MEAN
    p.y_begin, p.y_end = 0, 8
    for f in ("image_feats", "depth", "projection", "feature_size", "image_size"):
        setattr(p, f, 256)  # never dereferenced: validation fails first in every case below
    return p


def test_validation_status_codes():
    lib = _lib.load()
    fwd = lambda p: lib.fbev_forward(ctypes.byref(p), 256, None, None)
    assert lib.fbev_forward(None, 256, None, None) == 1          # FBEV_ERR_NULL
    p = _problem(); p.struct_size = 8
    assert fwd(p) == 2                                            # FBEV_ERR_STRUCT
    p = _problem(); p.C = 0
    assert fwd(p) == 3                                            # FBEV_ERR_SHAPE
    p = _problem(); p.proj_stride = 9
    assert fwd(p) == 3
    p = _problem(); p.y_end = 9
    assert fwd(p) == 3
    p = _problem(); p.D = 5                                       # parametric depth must have 2 channels
    assert fwd(p) == 3
    p = _problem(); p.dtype = 7
    assert fwd(p) == 4
    p = _problem(); p.out_dtype = _lib.BF16                       # output narrower than the features
    assert fwd(p) == 4                                            # FBEV_ERR_DTYPE
    p = _problem(); p.mode = 4
    assert fwd(p) == 5                                            # FBEV_ERR_MODE
    p = _problem(); p.mode = _lib.DEPTH_CATEGORICAL_LOGITS; p.depth_delta = 1.0   # logits need the statistics scratch
    assert fwd(p) == 1
    p = _problem(); p.mode = _lib.DEPTH_CATEGORICAL; p.depth_delta = 0.0
    assert fwd(p) == 5
    p = _problem(); p.image_feats = 258
    assert fwd(p) == 6
    p = _problem(); p.workspace = 264
    assert fwd(p) == 6                                            # FBEV_ERR_ALIGN
    p = _problem(); p.B = 1 << 20; p.H = 1 << 10; p.W = 1 << 10
    assert fwd(p) == 7                                            # FBEV_ERR_RANGE
    p = _problem(); p.image_feats = None
    assert fwd(p) == 1
    p = _problem()
    assert lib.fbev_forward(ctypes.byref(p), None, None, None) == 1
    # peer copies of the output: at most seven, none of them NULL, aligned like the output (checked before any launch)
    one = (ctypes.c_void_p * 1)(512)
    assert lib.fbev_forward_peers(ctypes.byref(p), 256, None, 1, None, None) == 3
    assert lib.fbev_forward_peers(ctypes.byref(p), 256, one, 8, None, None) == 3
    assert lib.fbev_forward_peers(ctypes.byref(p), 256, (ctypes.c_void_p * 1)(None), 1, None, None) == 1
    assert lib.fbev_forward_peers(ctypes.byref(p), 256, (ctypes.c_void_p * 1)(516), 1, None, None) == 6
    # the projection builder refuses missing arrays and empty batches
    assert lib.fbev_projection_matrices(None, 256, 256, 256, 256, 1, None) == 1
    assert lib.fbev_projection_matrices(256, 256, 256, 256, 256, 0, None) == 3
    assert _lib.strerror(99) == "unknown status"
    for code in range(0, 12):
        assert _lib.strerror(code) != "unknown status"


def test_backward_scratch_size_and_checks():
    lib = _lib.load()
    p = _problem()
    tex = 1 * 2 * 4 * 4
    assert lib.fbev_backward_min_scratch_bytes(ctypes.byref(p), 3) == 0        # float32: in place
    # the gradients' sort by texel: counters, a counter block, 4096 entries (the least capacity) of 36 bytes
    # (entry, grouped copy, position), 68 when they also carry the parametric depth gradient
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 1) == 256 + 256 + 4096 * 36
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 3) == 256 + 256 + 4096 * 68
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 2) == 256 + 256 + 4096 * 68
    p.dtype = p.out_dtype = _lib.BF16
    assert lib.fbev_backward_min_scratch_bytes(ctypes.byref(p), 3) == tex * 8 * 4 + tex * 2 * 4
    assert lib.fbev_backward_min_scratch_bytes(ctypes.byref(p), 1) == tex * 8 * 4
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 1) == tex * 8 * 4 + 256 + 256 + 4096 * 36
    # 16-bit gradients without scratch are refused before anything is launched
    assert lib.fbev_backward(ctypes.byref(p), 256, 256, 256, None, 0, 3, None) == 8   # FBEV_ERR_SCRATCH
    assert lib.fbev_backward(ctypes.byref(p), 256, 256, 256, None, 0, 0, None) == 0   # nothing requested
    # deterministic backward: 256-byte head + 64-bit fixed-point sums, whatever the element type
    det = _lib.BWD_DETERMINISTIC
    for dtype in (_lib.BF16, _lib.F32):
        p.dtype = p.out_dtype = dtype
        least = 256 + tex * 8 * 8 + tex * 2 * 8   # both gradients are always formed
        assert lib.fbev_backward_min_scratch_bytes(ctypes.byref(p), 3 | det) == least
        assert lib.fbev_backward_min_scratch_bytes(ctypes.byref(p), 2 | det) == least
        # + the entry lists of the feature gradient's sort (no depth values ride on them in this mode)
        assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 3 | det) == least + 256 + 256 + 4096 * 36
        assert lib.fbev_backward(ctypes.byref(p), 256, 256, 256, None, 0, 3 | det, None) == 8


def test_backward_scratch_of_large_feature_maps():
    """From 8192 texels per sample on, the texel counters are scanned into a second array (8 bytes per texel
    instead of 4) and the parametric depth gradient no longer rides on the entries (36 bytes per entry, not 68)."""
    lib = _lib.load()
    r256 = lambda n: (n + 255) // 256 * 256  # noqa: E731
    p = _problem()
    p.N, p.H, p.W = 2, 64, 64            # 8192 texels per sample
    p.X, p.Y, p.Z, p.y_end = 64, 64, 4, 64
    entries = p.X * p.Y * p.N * p.Z // 2
    cnt = r256((p.N * p.H * p.W + 1) * 4)
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 3) == cnt + 256 + entries * 36   # 8192 texels: one array
    p.H = 65                              # 8320 texels per sample
    cnt = r256((p.N * p.H * p.W + 1) * 4)
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 3) == 2 * cnt + 256 + entries * 36
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 2) == 0      # depth alone: no lists at this size
    p.H = 32                              # 4096 texels per sample: the depth gradient rides on the entries
    cnt = r256((p.N * p.H * p.W + 1) * 4)
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 3) == cnt + 256 + entries * 68
    p.B = 3                               # 12288 texels in the run of three samples: second array again
    cnt = r256((p.B * p.N * p.H * p.W + 1) * 4)
    assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), 3) == 2 * cnt + 256 + 3 * entries * 68


def test_operator_refuses_cpu_tensors():
    from flashbev_b200 import flash_bevpool
    from flashbev_b200 import synth
    inp = synth.make_inputs(synth.Workload("t", 1, 2, 8, 4, 4, 4, 8, 8, 2, 10.0, dtype="fp32"), "parametric")
    with pytest.raises(RuntimeError, match="CUDA"):
        flash_bevpool(**inp, depth_distribution=1)


def test_depth_spec_rules():
    from flashbev_b200 import DepthSpec
    assert int(DepthSpec(1)) == 1 and DepthSpec(1).pool == "mean"
    s = DepthSpec(2, depth_bin_range=(1.0, 0.5))
    assert s.pool == "sum" and (s.d0, s.delta) == (1.0, 0.5)
    with pytest.raises(ValueError):
        DepthSpec(2)
    assert DepthSpec(3, depth_bin_range=(1.0, 0.5)).pool == "sum"
    with pytest.raises(ValueError):
        DepthSpec(3)
    with pytest.raises(ValueError):
        DepthSpec(4)
    with pytest.raises(ValueError):
        DepthSpec(0, pool="max")


def test_drop_in_package_name_exports_the_reference_names():
    import flashbevpool
    assert sorted(flashbevpool.__all__) == ["FlashBEVPool", "SamplingVT", "flash_bevpool"]
