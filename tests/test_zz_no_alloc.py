"""GPU test of fbev_backward_static_scratch, the backward for callers that cannot allocate scratch.

A process that fixed its device-memory budget at start-up (or a plug-in whose host owns the memory
pool) cannot give fbev_backward the float32 scratch it needs for 16-bit gradients.  The entry point
under test keeps that scratch inside the library image.  Here it is called through the C ABI twice in
a row, with different upstream gradients, and each result is compared with what fbev_backward
produces with caller-allocated scratch and with the CPU oracle: the second call shows that leftovers
of the first do not leak into it.  A float32 problem (which needs no scratch at all) goes through the
same entry point.  The size limit is checked too.  (Collected last on purpose: a run that stops at the first
failure has then already run every other test.)
"""
import ctypes

import numpy as np
import pytest
import torch

from flashbev_b200 import _lib, synth
from flashbev_b200.flash_bevpool import DepthSpec, make_problem
from oracle import oracle as O
from tests.helpers import TOL_F32, TOL_LOWP, host_threads, oracle_problem, rel_err, rel_err_quantised

pytestmark = pytest.mark.gpu


def _grads(lib, prob, keep, go, static):
    dev = keep[0].device
    g_feats = torch.full_like(keep[0], float("nan"))  # the call must overwrite every element
    g_depth = torch.full_like(keep[1], float("nan"))
    flags = _lib.BWD_FEATS | _lib.BWD_DEPTH
    stream = torch.cuda.current_stream(dev).cuda_stream
    if static:
        rc = lib.fbev_backward_static_scratch(ctypes.byref(prob), go.data_ptr(), g_feats.data_ptr(),
                                              g_depth.data_ptr(), flags, stream)
    else:
        need = lib.fbev_backward_scratch_bytes(ctypes.byref(prob), flags)
        scratch = torch.empty(need, dtype=torch.uint8, device=dev)
        rc = lib.fbev_backward(ctypes.byref(prob), go.data_ptr(), g_feats.data_ptr(), g_depth.data_ptr(),
                               scratch.data_ptr(), need, flags, stream)
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize(dev)
    return g_feats.float().cpu().numpy(), g_depth.float().cpu().numpy()


@pytest.mark.parametrize("dtype,mode", [("bf16", "categorical"), ("fp16", "parametric"), ("fp32", "categorical")])
def test_static_scratch_backward_matches_caller_scratch_backward(cuda_device, dtype, mode):
    lib = _lib.load()
    w = synth.Workload("noalloc", B=2, N=6, C=80, H=16, W=44, D=118, X=48, Y=40, Z=8, xy_extent=50.0, dtype=dtype,
                       seed=77, jitter=True)
    inp = {k: v.to(cuda_device) for k, v in synth.make_inputs(w, mode).items()}
    spec = DepthSpec(2, depth_bin_range=(w.d0, w.delta)) if mode == "categorical" else DepthSpec(1)
    prob, keep = make_problem(inp["depth_params"], inp["image_feats"], inp["projection_matrices"],
                              inp["feature_size"], inp["image_size"], inp["roi_range"], inp["grid_size"], spec,
                              1e-6, 0.0)
    need = lib.fbev_backward_min_scratch_bytes(ctypes.byref(prob), 3)
    assert (need == 0) if dtype == "fp32" else (0 < need <= _lib.STATIC_SCRATCH_BYTES)
    cpu = oracle_problem(inp, w, "categorical" if mode == "categorical" else "laplace")
    for call in range(2):  # two calls in a row share the built-in array
        go = synth.upstream_grad(w, seed_offset=call).to(device=cuda_device, dtype=keep[0].dtype)
        ref_f, ref_d = _grads(lib, prob, keep, go, static=False)
        got_f, got_d = _grads(lib, prob, keep, go, static=True)
        assert np.isfinite(got_f).all() and np.isfinite(got_d).all()
        # against the CPU oracle (float64 gradients of the same rounded inputs)
        ora_f, ora_d = O.backward(cpu, go.float().cpu().numpy(), dtype=np.float64, threads=host_threads())
        if dtype == "fp32":
            assert rel_err(got_f, ora_f) < TOL_F32 and rel_err(got_d, ora_d) < TOL_F32, f"call {call}: vs oracle"
            assert rel_err(got_f, ref_f) < TOL_F32 and rel_err(got_d, ref_d) < TOL_F32, f"call {call}"
            continue
        assert rel_err_quantised(got_f, ora_f, dtype) < TOL_LOWP, f"call {call}: d_feats vs oracle"
        assert rel_err_quantised(got_d, ora_d, dtype) < TOL_LOWP, f"call {call}: d_depth vs oracle"
        # both sides sum with unordered float32 atomics and round once to the 16-bit type: equal up to one
        # ulp of that type plus the suite's 16-bit tolerance
        assert rel_err_quantised(got_f, ref_f, dtype, ulps=1.0) < TOL_LOWP, f"call {call}: d_feats"
        assert rel_err_quantised(got_d, ref_d, dtype, ulps=1.0) < TOL_LOWP, f"call {call}: d_depth"
        assert np.abs(ref_f).max() > 0 and np.abs(ref_d).max() > 0


def test_static_scratch_backward_refuses_problems_beyond_its_limit(cuda_device):
    lib = _lib.load()
    w = synth.workload("cfg3", dtype="bf16")  # 4 x 6 x 32 x 88 texels: 53 MB of float32 scratch
    inp = {k: v.to(cuda_device) for k, v in synth.make_inputs(w, "categorical").items()}
    prob, keep = make_problem(inp["depth_params"], inp["image_feats"], inp["projection_matrices"],
                              inp["feature_size"], inp["image_size"], inp["roi_range"], inp["grid_size"],
                              DepthSpec(2, depth_bin_range=(w.d0, w.delta)), 1e-6, 0.0)
    assert lib.fbev_backward_min_scratch_bytes(ctypes.byref(prob), 3) > _lib.STATIC_SCRATCH_BYTES
    go = torch.zeros(w.B, w.Y, w.X, w.C, dtype=torch.bfloat16, device=cuda_device)
    g_feats, g_depth = torch.empty_like(keep[0]), torch.empty_like(keep[1])
    rc = lib.fbev_backward_static_scratch(ctypes.byref(prob), go.data_ptr(), g_feats.data_ptr(), g_depth.data_ptr(),
                                          3, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_STATIC_LIMIT
    assert "FBEV_STATIC_SCRATCH_BYTES" in _lib.strerror(rc)
    # one gradient alone (21.6 MB) is still too large; a float32 problem needs no scratch and is accepted
    assert lib.fbev_backward_static_scratch(ctypes.byref(prob), go.data_ptr(), g_feats.data_ptr(), None, 1,
                                            torch.cuda.current_stream().cuda_stream) == _lib.ERR_STATIC_LIMIT
