"""numpy front end of the CPU oracle (``fbev_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the test suite, the smoke check and the benchmark's CPU-baseline leg may import
this module.  It is the checker for the CUDA path, never a fallback for it.

The C library restates the reference operator's arithmetic
(flashbev/flashbevpool/src/flash_bevpool_cuda.cu:31-216 forward, :446-681 backward)
plus the categorical depth mode; see the header of ``fbev_oracle.c`` for the pinned
operation order and the pinning status of each mode.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfbev_oracle.so")

MODE_GAUSSIAN, MODE_LAPLACE, MODE_CATEGORICAL = 0, 1, 2
POOL_MEAN, POOL_SUM = 0, 1


class _Args(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int), ("N", ctypes.c_int), ("H", ctypes.c_int), ("W", ctypes.c_int),
        ("C", ctypes.c_int), ("D", ctypes.c_int),
        ("X", ctypes.c_int), ("Y", ctypes.c_int), ("Z", ctypes.c_int),
        ("proj_stride", ctypes.c_int),
        ("feats", ctypes.c_void_p), ("depth", ctypes.c_void_p), ("proj", ctypes.c_void_p),
        ("feature_size", ctypes.c_void_p),
        ("image_h", ctypes.c_int), ("image_w", ctypes.c_int),
        ("roi", ctypes.c_float * 6),
        ("eps", ctypes.c_float), ("threshold", ctypes.c_float),
        ("mode", ctypes.c_int), ("pool", ctypes.c_int),
        ("d0", ctypes.c_float), ("delta", ctypes.c_float),
        ("y_begin", ctypes.c_int), ("y_end", ctypes.c_int),
        ("threads", ctypes.c_int),
    ]


def build(force: bool = False) -> str:
    """Compile the oracle library with the Makefile beside it (gcc only)."""
    src = [os.path.join(_HERE, n) for n in ("fbev_oracle.c", "fbev_oracle_body.inc")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "libfbev_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        for name in ("fbev_oracle_forward_f32", "fbev_oracle_forward_f64"):
            getattr(_lib, name).argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_void_p]
            getattr(_lib, name).restype = ctypes.c_int
        for name in ("fbev_oracle_backward_f32", "fbev_oracle_backward_f64"):
            getattr(_lib, name).argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_void_p,
                                            ctypes.c_void_p, ctypes.c_int]
            getattr(_lib, name).restype = ctypes.c_int
        _lib.fbev_oracle_indices.argtypes = [ctypes.POINTER(_Args)] + [ctypes.c_void_p] * 5
        _lib.fbev_oracle_indices.restype = ctypes.c_int
        _lib.fbev_oracle_num_threads.restype = ctypes.c_int
    return _lib


def projection(sensor2ego, camera2imgs, post_rots, post_trans) -> np.ndarray:
    """[B,N,3,4] float64 matrices from float32 calibration arrays (sampling_vt.py:21-33)."""
    arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in (sensor2ego, camera2imgs, post_rots, post_trans)]
    B, N = arrs[1].shape[:2]
    out = np.empty((B, N, 3, 4), np.float64)
    f = lib().fbev_oracle_projection
    f.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int]
    f.restype = ctypes.c_int
    rc = f(*[a.ctypes.data for a in arrs], out.ctypes.data, B * N)
    if rc:
        raise ValueError("singular sensor2ego")
    return out


def host_threads() -> int:
    return int(lib().fbev_oracle_num_threads())


@dataclass
class Problem:
    """One operator call, as host arrays.  Layouts follow flash_bevpool.py:28-34."""
    feats: np.ndarray            # [B,N,H,W,C] float32 (pre-rounded for low-precision cases)
    depth: np.ndarray            # [B,N,H,W,2] or [B,N,H,W,D] float32
    proj: np.ndarray             # [B,N,3,4] or [B,N,4,4] float32
    image_size: Tuple[int, int]  # (image_h, image_w)
    roi: Sequence[float]         # xmin,xmax,ymin,ymax,zmin,zmax
    grid: Tuple[int, int, int]   # X, Y, Z
    mode: int = MODE_LAPLACE
    pool: Optional[int] = None   # default: mean for parametric, sum for categorical
    eps: float = 1e-6
    threshold: float = 1e-6
    d0: float = 1.0
    delta: float = 1.0
    feature_size: Optional[np.ndarray] = None  # [B,N,2] int32, default (H, W)
    y_range: Optional[Tuple[int, int]] = None
    _keep: list = field(default_factory=list, repr=False)

    def args(self, threads: int = 1) -> _Args:
        f = np.ascontiguousarray(self.feats, dtype=np.float32)
        d = np.ascontiguousarray(self.depth, dtype=np.float32)
        p = np.ascontiguousarray(self.proj, dtype=np.float32)
        B, N, H, W, C = f.shape
        fs = self.feature_size
        if fs is None:
            fs = np.tile(np.array([H, W], dtype=np.int32), (B, N, 1))
        fs = np.ascontiguousarray(fs, dtype=np.int32)
        self._keep = [f, d, p, fs]
        a = _Args()
        a.B, a.N, a.H, a.W, a.C, a.D = B, N, H, W, C, d.shape[-1]
        a.X, a.Y, a.Z = (int(v) for v in self.grid)
        a.proj_stride = int(p.shape[-1] * p.shape[-2])
        a.feats, a.depth, a.proj = f.ctypes.data, d.ctypes.data, p.ctypes.data
        a.feature_size = fs.ctypes.data
        a.image_h, a.image_w = int(self.image_size[0]), int(self.image_size[1])
        a.roi = (ctypes.c_float * 6)(*[float(np.float32(v)) for v in self.roi])
        a.eps, a.threshold = float(self.eps), float(self.threshold)
        a.mode = int(self.mode)
        pool = self.pool
        if pool is None:
            pool = POOL_SUM if self.mode == MODE_CATEGORICAL else POOL_MEAN
        a.pool = int(pool)
        a.d0, a.delta = float(self.d0), float(self.delta)
        yb, ye = self.y_range if self.y_range is not None else (0, a.Y)
        a.y_begin, a.y_end = int(yb), int(ye)
        a.threads = int(threads)
        return a

    @property
    def out_shape(self):
        B, _, _, _, C = self.feats.shape
        return (B, self.grid[1], self.grid[0], C)


def forward(p: Problem, dtype=np.float32, threads: int = 1, with_count: bool = False):
    """BEV features [B,Y,X,C] (rows outside ``y_range`` stay zero) and optionally the count [B,Y,X]."""
    a = p.args(threads)
    out = np.zeros(p.out_shape, dtype=dtype)
    cnt = np.zeros(p.out_shape[:3], dtype=np.int32)
    fn = lib().fbev_oracle_forward_f32 if dtype == np.float32 else lib().fbev_oracle_forward_f64
    rc = fn(ctypes.byref(a), out.ctypes.data, cnt.ctypes.data)
    assert rc == 0
    return (out, cnt) if with_count else out


def backward(p: Problem, grad_out: np.ndarray, dtype=np.float32, threads: int = 1,
             legacy_depth_grad: bool = False):
    """(d_feats [B,N,H,W,C], d_depth [B,N,H,W,D]) for an upstream gradient [B,Y,X,C]."""
    a = p.args(threads)
    go = np.ascontiguousarray(grad_out, dtype=np.float32)
    assert go.shape == p.out_shape
    d_feats = np.zeros(p.feats.shape, dtype=dtype)
    d_depth = np.zeros(p.depth.shape, dtype=dtype)
    fn = lib().fbev_oracle_backward_f32 if dtype == np.float32 else lib().fbev_oracle_backward_f64
    rc = fn(ctypes.byref(a), go.ctypes.data, d_feats.ctypes.data, d_depth.ctypes.data,
            int(bool(legacy_depth_grad)))
    assert rc == 0
    return d_feats, d_depth


def indices(p: Problem):
    """Integer decisions of every (b, n, y, x, z) candidate and the per-cell count.

    Returns dict(u0, v0, kbin: int32 [B,N,Y,X,Z]; valid: uint8 [B,N,Y,X,Z]; count: int32 [B,Y,X]).
    """
    a = p.args(1)
    shp = (a.B, a.N, a.Y, a.X, a.Z)
    u0 = np.empty(shp, np.int32)
    v0 = np.empty(shp, np.int32)
    kb = np.empty(shp, np.int32)
    va = np.empty(shp, np.uint8)
    cnt = np.empty((a.B, a.Y, a.X), np.int32)
    rc = lib().fbev_oracle_indices(ctypes.byref(a), u0.ctypes.data, v0.ctypes.data, kb.ctypes.data,
                                   va.ctypes.data, cnt.ctypes.data)
    assert rc == 0
    return {"u0": u0, "v0": v0, "kbin": kb, "valid": va, "count": cnt}


def softmax_bins(logits, dtype=np.float64):
    """Softmax over the last axis (the depth bins), evaluated in ``dtype``: what a model's depth head applies before
    the operator, and what the operator's logits mode folds into its lookup."""
    l = np.asarray(logits, dtype)
    e = np.exp(l - l.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def softmax_bins_backward(prob, d_prob):
    """Gradient with respect to the logits from the gradient with respect to the probabilities:
    p_k * (g_k - sum_j g_j p_j) per texel."""
    p = np.asarray(prob, np.float64)
    g = np.asarray(d_prob, np.float64)
    return p * (g - (g * p).sum(axis=-1, keepdims=True))


def pillar_pool(depth, feat, u, v, z, batch_camera, ranks, starts, lengths, n_cells, laplace, epsilon=1e-6,
                dtype=np.float64):
    """Pillar pooling over pre-sorted sample lists, restating sampling_vt_pillarpool_fused_kernel
    (flashbev/flashbevpool/src/sampling_vt_cuda.cu:24-127) with numpy: depth [BN,h,w,2], feat [BN,h,w,C], flat
    per-sample u, v (feature-map coordinates), z (camera depth), camera index, BEV cell rank; per interval its
    first sample and length.  Returns [n_cells, C]: the mean over each interval's accepted samples, zero
    elsewhere.  Parity: pinned through the module fixtures (the dense branch of the reference module computes
    the same mean when no weight threshold is set)."""
    depth = np.asarray(depth, dtype)
    feat = np.asarray(feat, dtype)
    u, v, z = (np.asarray(a, dtype) for a in (u, v, z))
    cam = np.asarray(batch_camera, np.int64)
    h, w = depth.shape[1:3]
    ok = (u >= 0) & (u < w) & (v >= 0) & (v < h) & (z > 0)                     # :65-67
    u0 = np.floor(u).astype(np.int64).clip(0, w - 1)
    v0 = np.floor(v).astype(np.int64).clip(0, h - 1)
    u1, v1 = np.minimum(u0 + 1, w - 1), np.minimum(v0 + 1, h - 1)
    wu, wv = u - u0, v - v0
    wts = [((1 - wu) * (1 - wv), v0, u0), (wu * (1 - wv), v0, u1), ((1 - wu) * wv, v1, u0), (wu * wv, v1, u1)]
    par = sum(wt[:, None] * depth[cam, vv, uu] for wt, vv, uu in wts)          # :89-97
    f = sum(wt[:, None] * feat[cam, vv, uu] for wt, vv, uu in wts)             # :104-107
    mean, sigma = par[:, 0], par[:, 1]
    zs = (z - mean) / (sigma + epsilon)
    wgt = 0.5 * np.exp(-np.abs(zs)) / (sigma + epsilon) if laplace else np.exp(-0.5 * zs * zs) / (sigma + epsilon)
    wgt = np.where(ok, wgt, 0.0)
    interval = np.repeat(np.arange(len(starts)), np.asarray(lengths, np.int64))
    acc = np.zeros((len(starts), feat.shape[-1]), dtype)
    np.add.at(acc, interval, wgt[:, None] * f)
    cnt = np.bincount(interval, weights=ok.astype(dtype), minlength=len(starts))
    out = np.zeros((n_cells, feat.shape[-1]), dtype)
    cells = np.asarray(ranks, np.int64)[np.asarray(starts, np.int64)]
    out[cells] = np.where(cnt[:, None] > 0, acc / np.maximum(cnt, 1)[:, None], 0.0)
    return out
