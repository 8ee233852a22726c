"""Bitwise reproducible backward (``deterministic=True`` -> FBEV_BWD_DETERMINISTIC of the C ABI).

Two ways lead to the fixed-point sums: large problems whose channel rows are whole 16-byte chunks go through the
default pipeline's kernels (list phase + entries, sort by texel, gather) in their fixed-point instantiations, all
others through a one-cell-per-warp kernel.  The small shapes below take the second way by themselves and the first
one under the tuning switch that forces the sort.

Two things are checked on the GPU: the gradients of repeated runs are equal bit for bit (the default path adds
float32 values in arrival order and is not), and they meet the same bars against the CPU oracle as the default
path: float32 within 1e-5, 16-bit types within 2e-3 beyond their one rounding, as max|a-b| / max|b| per tensor.
"""
import ctypes

import numpy as np
import pytest
import torch

from flashbev_b200 import _lib, flash_bevpool, synth
from flashbev_b200.flash_bevpool import DepthSpec, make_problem
from oracle import oracle as O
from tests.helpers import (SMALL, TOL_F32, TOL_LOWP, host_threads, op_kwargs, oracle_problem, rel_err,
                           rel_err_quantised, to_device, tuning)

pytestmark = pytest.mark.gpu


def grads(inp, device, go, **kw):
    dev = to_device(inp, device)
    dev["image_feats"].requires_grad_(True)
    dev["depth_params"].requires_grad_(True)
    flash_bevpool(**dev, **kw).backward(go.to(device))
    torch.cuda.synchronize()
    return dev["image_feats"].grad, dev["depth_params"].grad


def deterministic_case(w, mode, device, report, pool=None, dtype=None, legacy=False, threshold=0.0, repeats=3, y_range=None):
    name = dtype or w.dtype
    inp = synth.make_inputs(w, "categorical" if mode == "categorical" else "parametric", dtype=dtype)
    go = synth.upstream_grad(w)
    if name != "fp32":
        go = go.to(inp["image_feats"].dtype)
    if y_range is not None:  # the rows outside the range receive no gradient
        masked = torch.zeros_like(go)
        masked[:, y_range[0]:y_range[1]] = go[:, y_range[0]:y_range[1]]
        go = masked
    p = oracle_problem(inp, w, mode, pool=pool, threshold=threshold, y_range=y_range)
    rf, rd = O.backward(p, go.float().numpy(), dtype=np.float64, legacy_depth_grad=legacy, threads=host_threads())
    kw = dict(op_kwargs(w, mode, threshold, pool, y_range), legacy_depth_grad=legacy, deterministic=True)
    runs = [grads(inp, device, go, **kw) for _ in range(repeats)]
    for gf, gd in runs[1:]:
        assert torch.equal(gf, runs[0][0]), "feature gradients of two runs differ"
        assert torch.equal(gd, runs[0][1]), "depth gradients of two runs differ"
    gf, gd = runs[0]
    assert gf.dtype == inp["image_feats"].dtype and gd.dtype == inp["depth_params"].dtype
    tol = TOL_F32 if name == "fp32" else TOL_LOWP
    for label, a, b in (("d_feats", gf, rf), ("d_depth", gd, rd)):
        a = a.float().cpu().numpy()
        err = rel_err(a, b) if name == "fp32" else rel_err_quantised(a, b, name)
        report(f"deterministic {w.name} {mode} {name} {label}: {err:.3e} (bar {tol:g}), {repeats} runs bit-identical")
        assert err < tol, f"{w.name} {mode} {label}: {err:.3e} >= {tol}"


@pytest.mark.parametrize("mode", ["gaussian", "laplace", "categorical"])
@pytest.mark.parametrize("pool", ["mean", "sum"])
def test_small_shapes_every_mode_and_pooling(cuda_device, parity_report, mode, pool):
    deterministic_case(SMALL, mode, cuda_device, parity_report, pool=pool)


@pytest.mark.parametrize("mode", ["gaussian", "laplace", "categorical"])
def test_small_shapes_through_the_sorted_pipeline(cuda_device, parity_report, mode):
    lib = _lib.load()
    with tuning(lib, 0, 0, 0, 0, 7):
        deterministic_case(SMALL, mode, cuda_device, parity_report, pool="mean")
        deterministic_case(SMALL, mode, cuda_device, parity_report, pool="sum", dtype="bf16")
        deterministic_case(SMALL, mode, cuda_device, parity_report, legacy=mode != "categorical", threshold=1e-3, dtype="fp16")


def test_full_entry_list_changes_no_bit(cuda_device):
    """With room for only 4096 entries nearly every warp finds the list full and adds its records itself; which
    warps do depends on the order they arrive in.  Every term is formed the same way on both routes, so the
    gradients must equal those of a run with room for all entries, bit for bit, and each other."""
    lib = _lib.load()
    w = synth.workload("cfg3", B=2, X=96, Y=80)
    for mode, dtype in (("categorical", "bf16"), ("laplace", "fp32")):
        inp = synth.make_inputs(w, "categorical" if mode == "categorical" else "parametric", dtype=dtype)
        go = synth.upstream_grad(w).to(inp["image_feats"].dtype)
        kw = dict(op_kwargs(w, mode), deterministic=True)
        with tuning(lib, 0, 0, 0, 0, 7):
            roomy = grads(inp, cuda_device, go, **kw)
        with tuning(lib, 0, 0, 0, 0, 8):
            tight = [grads(inp, cuda_device, go, **kw) for _ in range(2)]
        for gf, gd in tight:
            assert torch.equal(gf, roomy[0]) and torch.equal(gd, roomy[1]), mode


def test_legacy_depth_gradient_threshold_and_row_range(cuda_device, parity_report):
    deterministic_case(SMALL, "laplace", cuda_device, parity_report, legacy=True)
    deterministic_case(SMALL, "gaussian", cuda_device, parity_report, threshold=1e-3)
    deterministic_case(SMALL, "categorical", cuda_device, parity_report, y_range=(4, 15))


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_sixteen_bit_types(cuda_device, parity_report, dtype):
    deterministic_case(synth.workload("cfg3", B=2, X=96, Y=80), "categorical", cuda_device, parity_report, dtype=dtype)
    deterministic_case(SMALL, "laplace", cuda_device, parity_report, dtype=dtype)


@pytest.mark.parametrize("C,dtype", [(5, "fp32"), (12, "bf16"), (33, "fp16")])
def test_channel_counts_without_16_byte_rows(cuda_device, parity_report, C, dtype):
    w = synth.Workload(f"odd{C}", B=2, N=5, C=C, H=8, W=22, D=16, X=24, Y=20, Z=4, xy_extent=25.6, d0=1.0, delta=2.0,
                       dtype=dtype, seed=40 + C, jitter=True)
    deterministic_case(w, "categorical", cuda_device, parity_report)
    deterministic_case(w, "gaussian", cuda_device, parity_report)


def test_many_height_bins_take_several_passes(cuda_device, parity_report):
    w = synth.Workload("tall", B=1, N=6, C=16, H=8, W=22, D=24, X=30, Y=30, Z=40, xy_extent=30.0, d0=1.0, delta=1.5,
                       dtype="fp32", seed=32)
    deterministic_case(w, "categorical", cuda_device, parity_report, pool="mean")
    deterministic_case(w, "laplace", cuda_device, parity_report)


def test_headline_and_training_shapes_at_full_size(cuda_device, parity_report):
    """cfg2 (bfloat16, one sample) and cfg3 (float32, four samples with their own rigs)."""
    deterministic_case(synth.workload("cfg2"), "categorical", cuda_device, parity_report)
    deterministic_case(synth.workload("cfg3"), "categorical", cuda_device, parity_report, repeats=2)
    deterministic_case(synth.workload("cfg3"), "laplace", cuda_device, parity_report, repeats=2)


def test_batch_taken_in_several_runs(cuda_device, parity_report):
    """Five samples whose entry lists would need 2.2 times the scratch budget go through the sort in runs of two, two
    and one sample; the fixed-point sums of the whole batch live side by side and must not notice."""
    w = synth.Workload("budget", B=5, N=6, C=16, H=8, W=22, D=24, X=256, Y=256, Z=16, xy_extent=40.0, d0=1.0,
                       delta=2.5, dtype="bf16", seed=61, jitter=True)
    assert w.X * w.Y * w.N * w.Z // 2 * 36 * w.B > 2 * _lib.SORT_BUDGET_BYTES
    deterministic_case(w, "categorical", cuda_device, parity_report, pool="mean", repeats=2)


def test_logits_mode(cuda_device, parity_report):
    """depth_distribution=3: the chain through the folded softmax is reproducible too."""
    w = synth.Workload("small", B=2, N=6, C=16, H=8, W=22, D=24, X=40, Y=36, Z=5, xy_extent=30.0, d0=1.0, delta=1.5,
                       dtype="fp32", seed=21, jitter=True)
    inp = synth.make_inputs(w, "categorical")
    g = torch.Generator().manual_seed(77)
    logits = torch.randn(inp["depth_params"].shape, generator=g) * 2.0
    prob = O.softmax_bins(logits.numpy())
    cpu = oracle_problem(dict(inp, depth_params=torch.from_numpy(prob.astype(np.float32))), w, "categorical", pool="sum")
    go = synth.upstream_grad(w)
    rf, rd_prob = O.backward(cpu, go.numpy(), dtype=np.float64, threads=host_threads())
    rd = O.softmax_bins_backward(prob, rd_prob)
    kw = dict(depth_distribution=3, depth_bin_range=(w.d0, w.delta), depth_weight_threshold=0.0, pool="sum",
              deterministic=True)
    a = grads(dict(inp, depth_params=logits), cuda_device, go, **kw)
    b = grads(dict(inp, depth_params=logits), cuda_device, go, **kw)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    ef, ed = rel_err(a[0].cpu().numpy(), rf), rel_err(a[1].cpu().numpy(), rd)
    parity_report(f"deterministic logits mode: d_feats {ef:.3e}, d_logits {ed:.3e} (bar {TOL_F32:g})")
    assert ef < TOL_F32 and ed < TOL_F32


def test_only_the_requested_gradient(cuda_device):
    w = SMALL
    inp = synth.make_inputs(w, "categorical")
    go = synth.upstream_grad(w)
    kw = dict(op_kwargs(w, "categorical"), deterministic=True)
    both = grads(inp, cuda_device, go, **kw)
    for k, ref in (("image_feats", both[0]), ("depth_params", both[1])):
        dev = to_device(inp, cuda_device)
        dev[k].requires_grad_(True)
        flash_bevpool(**dev, **kw).backward(go.to(cuda_device))
        assert torch.equal(dev[k].grad, ref)


def test_more_than_32_cameras_are_refused(cuda_device):
    w = synth.Workload("many", B=1, N=33, C=8, H=4, W=6, D=8, X=8, Y=8, Z=2, xy_extent=10.0, d0=1.0, delta=2.0,
                       dtype="fp32", seed=3)
    inp = to_device(synth.make_inputs(w, "categorical"), cuda_device)
    inp["image_feats"].requires_grad_(True)
    out = flash_bevpool(**inp, **op_kwargs(w, "categorical"), deterministic=True)
    with pytest.raises((RuntimeError, ValueError)):
        out.sum().backward()


def test_scratch_sizes_of_the_c_abi(cuda_device):
    """Least scratch: 256 bytes + 8 per element of both gradients (rounded up to 256 each; both are always formed),
    + 4 per depth element for logits; the entry lists of the sort come on top; less than the least is refused."""
    w = SMALL
    inp = to_device(synth.make_inputs(w, "categorical"), cuda_device)
    lib = _lib.load()
    p, keep = make_problem(inp["depth_params"], inp["image_feats"], inp["projection_matrices"], inp["feature_size"],
                           inp["image_size"], inp["roi_range"], inp["grid_size"],
                           DepthSpec(2, depth_bin_range=(w.d0, w.delta)), 1e-6, 0.0)
    tex = w.B * w.N * w.H * w.W
    r256 = lambda n: (n + 255) // 256 * 256  # noqa: E731
    least = 256 + r256(tex * w.C * 8) + r256(tex * w.D * 8)
    for flags in (_lib.BWD_FEATS | _lib.BWD_DEPTH, _lib.BWD_FEATS, _lib.BWD_DEPTH):
        assert lib.fbev_backward_min_scratch_bytes(ctypes.byref(p), flags | _lib.BWD_DETERMINISTIC) == least
        lists = lib.fbev_backward_scratch_bytes(ctypes.byref(p), _lib.BWD_FEATS) \
            - lib.fbev_backward_min_scratch_bytes(ctypes.byref(p), _lib.BWD_FEATS)
        assert lib.fbev_backward_scratch_bytes(ctypes.byref(p), flags | _lib.BWD_DETERMINISTIC) == least + lists
    only_f = _lib.BWD_FEATS | _lib.BWD_DETERMINISTIC
    go = synth.upstream_grad(w).to(cuda_device)
    gf = torch.empty_like(inp["image_feats"])
    small = torch.empty(1024, dtype=torch.uint8, device=cuda_device)
    rc = lib.fbev_backward(ctypes.byref(p), go.data_ptr(), gf.data_ptr(), None, small.data_ptr(), small.numel(), only_f,
                           torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_SCRATCH, _lib.strerror(rc)
    # the least scratch alone is enough (one-cell-per-warp kernel), and gives what the full scratch gives on this
    # small shape, which takes that kernel anyway
    ok = torch.empty(least, dtype=torch.uint8, device=cuda_device)
    rc = lib.fbev_backward(ctypes.byref(p), go.data_ptr(), gf.data_ptr(), None, ok.data_ptr(), ok.numel(), only_f,
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.strerror(rc)
    ref = grads(synth.make_inputs(w, "categorical"), cuda_device, synth.upstream_grad(w),
                **dict(op_kwargs(w, "categorical"), deterministic=True))[0]
    torch.cuda.synchronize()
    assert torch.equal(gf, ref)
