"""Shared pieces of the parity tests: problem construction for the CPU oracle and the CUDA
operator from the same seeded inputs, and the error measure the tolerances refer to."""
import contextlib
import glob
import os
import threading

import numpy as np
import torch

from flashbev_b200 import synth
from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")



@contextlib.contextmanager
def tuning(lib, *values):
    """fbev_set_tuning(*values) for the calls inside the block, put back to zeros after it.  The tuning is kept per
    host thread, and autograd normally runs a CUDA operator's backward on a worker thread of its own, which would
    not see it: inside the block autograd's worker threads are off, so the backward runs on the calling thread
    (checked with a probe function)."""
    class _Probe(torch.autograd.Function):
        ident = None

        @staticmethod
        def forward(ctx, x):
            return x.clone()

        @staticmethod
        def backward(ctx, g):
            _Probe.ident = threading.get_ident()
            return g

    with torch.autograd.set_multithreading_enabled(False):
        if torch.cuda.is_available():
            x = torch.ones(1, device="cuda", requires_grad=True)
            _Probe.apply(x).sum().backward()
            assert _Probe.ident == threading.get_ident(), "autograd ran the backward on another thread"
        lib.fbev_set_tuning(*values)
        try:
            yield
        finally:
            lib.fbev_set_tuning(0, 0, 0, 0, 0)

# Tolerances (relative error = max|a-b| / max|b| per tensor):
TOL_F32 = 1e-5       # float32 kernels vs the float32/float64 oracle
TOL_LOWP = 2e-3      # bfloat16 / float16 kernels vs the oracle on the same rounded inputs
TOL_DENSE = 5e-5     # oracle vs the reference's dense PyTorch path (grid_sample re-normalises coordinates)


def host_threads():
    """Threads the CPU oracle may use in the full-size cases (its results do not depend on the count: the
    float32 forward is sequential per cell, the float64 gradients are compared at 1e-5)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = np.abs(b).max()
    return float(np.abs(a - b).max() / (denom if denom > 0 else 1.0))


_MANTISSA_BITS = {"bf16": 7, "fp16": 10}


def rel_err_quantised(a, b, dtype_name, ulps=0.5):
    """Relative error of a result that was rounded to a 16-bit type, after setting aside that one
    rounding: max(|a-b| - half_ulp(b), 0) / max|b|.  A bfloat16 result cannot be closer than half an ulp
    (up to 2^-8 = 3.9e-3 of its value) to an unrounded reference, so that part is not an error of the kernel.
    ``ulps`` = 0.5 for a rounded result against an unrounded reference, 1.0 for two rounded results."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    mag = np.maximum(np.abs(b), 2.0 ** -24)
    half_ulp = ulps * 2.0 ** (np.floor(np.log2(mag)) - _MANTISSA_BITS[dtype_name])
    denom = np.abs(b).max()
    return float(np.maximum(np.abs(a - b) - half_ulp, 0.0).max() / (denom if denom > 0 else 1.0))


MODES = {"gaussian": O.MODE_GAUSSIAN, "laplace": O.MODE_LAPLACE, "categorical": O.MODE_CATEGORICAL}


def oracle_problem(inp, w, mode, threshold=0.0, pool=None, y_range=None, eps=1e-6):
    """Oracle problem from operator inputs (tensors of any float dtype are widened exactly)."""
    return O.Problem(
        feats=inp["image_feats"].float().cpu().numpy(), depth=inp["depth_params"].float().cpu().numpy(),
        proj=inp["projection_matrices"].float().cpu().numpy(),
        image_size=tuple(int(v) for v in inp["image_size"].tolist()),
        roi=[float(v) for v in inp["roi_range"].tolist()], grid=tuple(int(v) for v in inp["grid_size"].tolist()),
        mode=MODES[mode], pool=None if pool is None else (O.POOL_SUM if pool == "sum" else O.POOL_MEAN),
        eps=eps, threshold=threshold, d0=w.d0, delta=w.delta,
        feature_size=inp["feature_size"].cpu().numpy(), y_range=y_range)


def op_kwargs(w, mode, threshold=0.0, pool=None, y_range=None):
    kw = dict(depth_distribution={"gaussian": 0, "laplace": 1, "categorical": 2}[mode],
              depth_weight_threshold=threshold, epsilon=1e-6)
    if mode == "categorical":
        kw["depth_bin_range"] = (w.d0, w.delta)
    if pool is not None:
        kw["pool"] = pool
    if y_range is not None:
        kw["y_range"] = y_range
    return kw


def to_device(inp, device):
    return {k: v.to(device) for k, v in inp.items()}


def inputs_for(w, mode):
    return synth.make_inputs(w, "categorical" if mode == "categorical" else "parametric")


def golden_files():
    """Operator fixtures (the calibration fixture projection_*.npz is read by projection_golden)."""
    return sorted(f for f in glob.glob(os.path.join(GOLDEN, "*.npz"))
                  if not os.path.basename(f).startswith(("projection_", "module_")))


def projection_golden():
    """Calibration arrays and the matrices the reference's create_projection_matrix made of them."""
    return dict(np.load(os.path.join(GOLDEN, "projection_synthetic.npz")))


MODULE_GRID = {"x": [-20.0, 20.0, 1.0], "y": [-16.0, 16.0, 1.0], "z": [-4.0, 2.0, 1.0], "depth": [1.0, 60.0, 1.0]}
MODULE_INPUT_NAMES = ("x", "sensor2ego", "ego2global", "camera2imgs", "post_rots", "post_trans", "bda")


def module_golden(dist):
    """A recorded run of the reference's own SamplingVT module, dense branch (tests/golden/make_golden.py,
    module_case): the input list, the state of the two 1x1 heads, the BEV output and the depth head's output."""
    g = np.load(os.path.join(GOLDEN, f"module_dense_{dist}.npz"))
    inputs = [torch.from_numpy(g[f"in_{n}"]) for n in MODULE_INPUT_NAMES]
    state = {k[len("state_"):]: torch.from_numpy(g[k]) for k in g.files if k.startswith("state_")}
    return inputs, state, tuple(int(v) for v in g["image"]), g["bev"], g["depths"]


def harness_metrics(out, ref):
    """The figures the reference's parity harness judges by (tools/profile_differences.py:17-67, 70-127):
    MSE < 1e-6, MAE < 1e-6, mean of |diff| / max(|ref|, 1e-8) < 1e-3, cosine > 0.9999."""
    a = np.asarray(out, np.float64).ravel()
    b = np.asarray(ref, np.float64).ravel()
    diff = np.abs(a - b)
    return {"mse": float((diff ** 2).mean()), "mae": float(diff.mean()),
            "mean_rel": float((diff / np.maximum(np.abs(b), 1e-8)).mean()),
            "cos": float((a * b).sum() / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))}


def harness_pass(m):
    return m["mse"] < 1e-6 and m["mae"] < 1e-6 and m["mean_rel"] < 1e-3 and m["cos"] > 0.9999


def golden_problem(g):
    return O.Problem(g["feats"], g["depth"], g["proj"], tuple(int(v) for v in g["image_size"]),
                     [float(v) for v in g["roi"]], tuple(int(v) for v in g["grid"]),
                     mode=O.MODE_LAPLACE if int(g["laplace"]) else O.MODE_GAUSSIAN, threshold=float(g["threshold"]))


def golden_inputs(g, device):
    B, N, H, W, _ = g["feats"].shape
    return dict(
        image_feats=torch.from_numpy(g["feats"]).to(device), depth_params=torch.from_numpy(g["depth"]).to(device),
        projection_matrices=torch.from_numpy(g["proj"]).to(device),
        feature_size=torch.tensor([[H, W]], dtype=torch.int32).repeat(B * N, 1).view(B, N, 2).to(device),
        image_size=torch.from_numpy(g["image_size"]).to(device), roi_range=torch.from_numpy(g["roi"]).to(device),
        grid_size=torch.from_numpy(g["grid"]).to(device))


SMALL = synth.Workload("small", B=2, N=6, C=16, H=8, W=22, D=24, X=40, Y=36, Z=5, xy_extent=30.0,
                       d0=1.0, delta=1.5, dtype="fp32", seed=21, jitter=True)
