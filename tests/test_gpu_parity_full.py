"""GPU parity at the full sizes of the benchmark configurations: the training shape (cfg3), the multi-GPU batch
shape with per-sample rigs (cfg4, eight samples) and the large grid with 256 channels (cfg5).  Forward and both
gradients of the CUDA operator (ctypes -> C ABI of libfbev.so) against the CPU oracle on the same seeded inputs,
and the training shape against the reference's own CUDA kernels where a built copy exists.

Bars: float32 within 1e-5, bfloat16 within 2e-3, as max|a-b| / max|b| per tensor; per-cell sample counts
bit-exact.  For results stored in a 16-bit type the bar applies beyond the one rounding to that type
(helpers.rel_err_quantised); the plain figure is reported beside it in the run's "parity figures" section.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from flashbev_b200 import flash_bevpool, forward_with_count, synth
from oracle import oracle as O
from tests.helpers import (TOL_F32, TOL_LOWP, host_threads, inputs_for, op_kwargs, oracle_problem, rel_err,
                           rel_err_quantised, to_device)

pytestmark = pytest.mark.gpu

CFG3 = synth.workload("cfg3")
CFG4 = synth.workload("cfg4", B=8)
CFG5 = synth.workload("cfg5")


def full_case(w, mode, device, report, pool=None, threshold=0.0):
    """Forward + both gradients at full size against the oracle (float32 pinned order forward, float64 gradients)."""
    threads = host_threads()
    inp = inputs_for(w, mode)
    lowp = w.dtype != "fp32"
    go = synth.upstream_grad(w)
    if lowp:
        go = go.to(inp["image_feats"].dtype)
    p = oracle_problem(inp, w, mode, pool=pool, threshold=threshold)
    ref, ref_cnt = O.forward(p, threads=threads, with_count=True)
    rf, rd = O.backward(p, go.float().numpy(), dtype=np.float64, threads=threads)

    dev = to_device(inp, device)
    kw = op_kwargs(w, mode, threshold, pool)
    out, cnt = forward_with_count(**dev, **kw)
    assert np.array_equal(cnt.cpu().numpy(), ref_cnt), "per-cell sample counts differ"
    dev["image_feats"].requires_grad_(True)
    dev["depth_params"].requires_grad_(True)
    out_t = flash_bevpool(**dev, **kw)
    out_t.backward(go.to(device))
    torch.cuda.synchronize()
    assert torch.equal(out_t.detach(), out)  # training and inference forward agree bit for bit
    got = {"out": (out.float().cpu().numpy(), ref),
           "d_feats": (dev["image_feats"].grad.float().cpu().numpy(), rf),
           "d_depth": (dev["depth_params"].grad.float().cpu().numpy(), rd)}
    tol = TOL_LOWP if lowp else TOL_F32
    for name, (a, b) in got.items():
        plain = rel_err(a, b)
        err = rel_err_quantised(a, b, w.dtype) if lowp else plain
        report(f"{w.name} B={w.B} {mode} {w.dtype} {name}: max|a-b|/max|b| = {plain:.3e}"
               + (f", beyond one {w.dtype} rounding = {err:.3e}" if lowp else "")
               + f" (bar {tol:g}; accepted samples {int(ref_cnt.sum())})")
        assert err < tol, f"{w.name} {mode} {name}: {err:.3e} >= {tol}"


@pytest.mark.parametrize("mode", ["categorical", "laplace", "gaussian"])
def test_training_shape_full_size(cuda_device, parity_report, mode):
    """cfg3: B=4 with per-sample rigs, float32, 32x88 feature maps, 200x200x8 grid."""
    full_case(CFG3, mode, cuda_device, parity_report)


@pytest.mark.parametrize("mode", ["categorical", "laplace"])
def test_batch_shape_eight_samples_with_their_own_rigs(cuda_device, parity_report, mode):
    """cfg4 with eight samples (what one of eight GPUs holds of the B=64 batch), bfloat16."""
    full_case(CFG4, mode, cuda_device, parity_report)


@pytest.mark.parametrize("mode", ["categorical", "laplace"])
def test_large_grid_full_size(cuda_device, parity_report, mode):
    """cfg5: 512x512x16 grid, 256 channels (32 chunks per texel), 32x88 map (more than 8192 texels: the
    gradient sort runs its separate scan kernel), bfloat16."""
    full_case(CFG5, mode, cuda_device, parity_report)


def test_large_grid_float32_output_meets_the_plain_bar(cuda_device, parity_report):
    """cfg5 forward with bfloat16 inputs and a float32 result: no rounding of the result, so the plain figure
    stands against the bar by itself."""
    w = CFG5
    inp = inputs_for(w, "categorical")
    ref = O.forward(oracle_problem(inp, w, "categorical"), threads=host_threads())
    out = flash_bevpool(**to_device(inp, cuda_device), **op_kwargs(w, "categorical"), out_dtype=torch.float32)
    err = rel_err(out.cpu().numpy(), ref)
    parity_report(f"cfg5 categorical bf16 inputs, float32 output: max|a-b|/max|b| = {err:.3e} (bar {TOL_LOWP:g})")
    assert err < 1e-5


# ---- the reference's own CUDA kernels on the training shape ----
REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                       "libflashbev_ref.so")


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="reference CUDA library was not built")
@pytest.mark.parametrize("dist", [1, 0])
def test_training_shape_against_reference_cuda_kernels(cuda_device, parity_report, dist):
    """cfg3 (float32, parametric depth, mean pooling: the reference's only mode) forward and backward with the
    reference kernel's own depth gradient, plus the number of cells on which the two disagree about having
    accepted any sample (a non-zero output row there, a positive count here)."""
    ref = ctypes.CDLL(REF_LIB)
    vp, i32, f32c = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    ref.flashbev_ref_forward.argtypes = [i32] * 7 + [f32c, f32c] + [vp] * 5 + [i32] * 3 + [f32c] * 6 + [vp]
    ref.flashbev_ref_backward.argtypes = [i32] * 5 + [f32c, f32c] + [vp] * 7 + [i32] * 3 + [vp, vp]
    w = CFG3
    mode = "laplace" if dist == 1 else "gaussian"
    inp = to_device(inputs_for(w, mode), cuda_device)
    roi = [float(v) for v in inp["roi_range"].tolist()]
    f32 = np.float32
    vs = [float((f32(roi[2 * i + 1]) - f32(roi[2 * i])) / f32(g)) for i, g in enumerate(w.grid)]
    thr = 1e-6
    out_ref = torch.zeros(w.B, w.Y, w.X, w.C, device=cuda_device)
    torch.cuda.synchronize()
    rc = ref.flashbev_ref_forward(out_ref.numel(), w.C, w.N, w.B, dist, 0, 0, 1e-6, thr,
                                  inp["depth_params"].data_ptr(), inp["image_feats"].data_ptr(),
                                  inp["projection_matrices"].data_ptr(), inp["feature_size"].data_ptr(),
                                  inp["image_size"].data_ptr(), w.X, w.Y, w.Z, vs[0], vs[1], vs[2], roi[0], roi[2],
                                  roi[4], out_ref.data_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    # the reference's second forward variant (optimize_z_precompute, flash_bevpool_cuda.cu:84-109) groups the
    # projection's additions differently: how far its two variants are apart is how sharply "the reference's
    # float32 result" is defined on this shape (image 512x1408, feature columns up to 88: an ulp of the
    # feature coordinate is 7.6e-6 of a texel)
    out_ref_z = torch.zeros_like(out_ref)
    rc = ref.flashbev_ref_forward(out_ref.numel(), w.C, w.N, w.B, dist, 0, 1, 1e-6, thr,
                                  inp["depth_params"].data_ptr(), inp["image_feats"].data_ptr(),
                                  inp["projection_matrices"].data_ptr(), inp["feature_size"].data_ptr(),
                                  inp["image_size"].data_ptr(), w.X, w.Y, w.Z, vs[0], vs[1], vs[2], roi[0], roi[2],
                                  roi[4], out_ref_z.data_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    kw = dict(depth_distribution=dist, depth_weight_threshold=thr)
    out, cnt = forward_with_count(**inp, **kw)
    err = rel_err(out.cpu().numpy(), out_ref.cpu().numpy())
    err_z = rel_err(out.cpu().numpy(), out_ref_z.cpu().numpy())
    spread = rel_err(out_ref_z.cpu().numpy(), out_ref.cpu().numpy())
    ref_has = (out_ref != 0).any(dim=-1)
    mism = int((ref_has != (cnt > 0)).sum())
    parity_report(f"cfg3 {mode} vs reference CUDA kernel: forward {err:.3e} (its z-precompute variant: {err_z:.3e}; "
                  f"the reference's two variants against each other: {spread:.3e}); cells whose 'any sample "
                  f"accepted' differs: {mism} of {cnt.numel()}")
    # Two float32 evaluations of this shape that round the geometry differently cannot be expected within 1e-5 of
    # each other: float32 rounding of the feature coordinates alone moves the result 1.2e-5 away from a float64
    # evaluation (tests/test_oracle.py::test_float32_geometry_rounding_floor_on_the_training_shape), so two of
    # them may be 2.4e-5 apart.  The kernel here is held to 1e-5 against the oracle's pinned order (above); against
    # the reference binary, whose contraction into fused multiply-adds is the compiler's, the bar is 3e-5.
    bar = 3e-5
    assert min(err, err_z) < bar, f"forward vs reference kernel: {err:.3e} / {err_z:.3e}, bar {bar:.1e}"
    assert mism == 0
    go = synth.upstream_grad(w).to(cuda_device)
    gd_ref = torch.zeros_like(inp["depth_params"])
    gf_ref = torch.zeros_like(inp["image_feats"])
    torch.cuda.synchronize()
    rc = ref.flashbev_ref_backward(out_ref.numel(), w.C, w.N, w.B, dist, 1e-6, thr, go.data_ptr(),
                                   inp["depth_params"].data_ptr(), inp["image_feats"].data_ptr(),
                                   inp["projection_matrices"].data_ptr(), inp["feature_size"].data_ptr(),
                                   inp["image_size"].data_ptr(), inp["roi_range"].data_ptr(), w.X, w.Y, w.Z,
                                   gd_ref.data_ptr(), gf_ref.data_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    inp["image_feats"].requires_grad_(True)
    inp["depth_params"].requires_grad_(True)
    flash_bevpool(**inp, **kw, legacy_depth_grad=True).backward(go)
    ef = rel_err(inp["image_feats"].grad.cpu().numpy(), gf_ref.cpu().numpy())
    ed = rel_err(inp["depth_params"].grad.cpu().numpy(), gd_ref.cpu().numpy())
    parity_report(f"cfg3 {mode} vs reference CUDA kernel: d_feats {ef:.3e}, d_depth (the kernel's own formula) {ed:.3e}")
    # both sides sum with float32 atomics in an order that changes from run to run (the reference once per
    # channel thread); its depth gradient alone moves by about 1e-5 between two of its own runs on the small
    # shape and sums 4 times as many terms per texel here.  The feature gradient inherits the forward's bar.
    assert ef < bar and ed < 1e-4, f"backward vs reference kernel: feats {ef:.3e} depth {ed:.3e}"
