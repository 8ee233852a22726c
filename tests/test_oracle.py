"""CPU tests of the oracle: against the reference-generated golden fixtures, against its own
float64 twin, on hand-checkable cases and through properties of the operator."""
import numpy as np
import pytest

from flashbev_b200 import synth
from oracle import oracle as O
from tests.helpers import projection_golden  # noqa: E402
from tests.helpers import (SMALL, TOL_DENSE, TOL_F32, golden_files, golden_problem, inputs_for, oracle_problem,
                           rel_err)


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1][:-4])
def test_oracle_matches_reference_dense_path(path):
    """Forward and analytic gradients vs the reference's dense PyTorch path and autograd through it."""
    g = np.load(path)
    p = golden_problem(g)
    out = O.forward(p)
    d_feats, d_depth = O.backward(p, g["grad_out"])
    assert rel_err(out, g["out"]) < TOL_DENSE
    assert rel_err(d_feats, g["d_feats"]) < TOL_DENSE
    assert rel_err(d_depth, g["d_depth"]) < TOL_DENSE
    # the reference's own acceptance test (tools/profile_differences.py:75-77,104)
    diff = out.astype(np.float64) - g["out"]
    assert (diff ** 2).mean() < 1e-6 and np.abs(diff).mean() < 1e-6
    cos = (out * g["out"]).sum() / (np.linalg.norm(out) * np.linalg.norm(g["out"]))
    assert cos > 0.9999


def test_golden_fixtures_exist():
    assert len(golden_files()) >= 5


@pytest.mark.parametrize("mode", ["gaussian", "laplace", "categorical"])
def test_f32_matches_f64_twin(mode):
    inp = inputs_for(SMALL, mode)
    p = oracle_problem(inp, SMALL, mode)
    assert rel_err(O.forward(p), O.forward(p, dtype=np.float64)) < TOL_F32
    go = synth.upstream_grad(SMALL).numpy()
    a = O.backward(p, go)
    b = O.backward(p, go, dtype=np.float64)
    assert rel_err(a[0], b[0]) < TOL_F32 and rel_err(a[1], b[1]) < TOL_F32


def _one_camera_problem(mode, depth, feats, **kw):
    # camera at the origin looking along +x: u = 8 - 8*y/x, v = 4 - 8*z/x on a 16x8 image, feature map 4x2... kept tiny
    P = np.array([[[[8.0, -8.0, 0.0, 0.0], [4.0, 0.0, -8.0, 0.0], [1.0, 0.0, 0.0, 0.0]]]], dtype=np.float32)
    return O.Problem(feats=feats, depth=depth, proj=P, image_size=(8, 16), roi=[0.0, 4.0, -2.0, 2.0, -1.0, 1.0],
                     grid=(2, 2, 1), mode=mode, threshold=0.0, **kw)


def test_hand_checked_single_sample():
    """One camera, one height bin: cell (x=1 -> vx=3, y=1 -> vy=1, z=0) projects to u=8-8/3, v=4."""
    H, W, C = 2, 4, 3
    feats = np.arange(H * W * C, dtype=np.float32).reshape(1, 1, H, W, C)
    depth = np.zeros((1, 1, H, W, 4), dtype=np.float32)
    depth[..., 1] = 0.25  # bin 1 = [2, 4) with d0=0, delta=2 holds d = 3
    p = _one_camera_problem(O.MODE_CATEGORICAL, depth, feats, d0=0.0, delta=2.0)
    out, cnt = O.forward(p, with_count=True)
    idx = O.indices(p)
    # feature coordinates: fu = (8 - 8/3)/16*4 = 4/3, fv = 4/8*2 = 1
    assert idx["u0"][0, 0, 1, 1, 0] == 1 and idx["v0"][0, 0, 1, 1, 0] == 1 and idx["kbin"][0, 0, 1, 1, 0] == 1
    du = 4.0 / 3.0 - 1.0
    f = lambda v, u: feats[0, 0, v, u]
    expect = 0.25 * ((1 - du) * f(1, 1) + du * f(1, 2))  # dv = 0; v1 clamps to the last row
    np.testing.assert_allclose(out[0, 1, 1], expect, rtol=1e-6)
    assert cnt[0, 1, 1] == 1
    # cell (x=0 -> vx=1, vy=1): u = 0, on the left border -> accepted with u0 = 0
    assert idx["valid"][0, 0, 1, 0, 0] == 1 and idx["u0"][0, 0, 1, 0, 0] == 0
    # vy = -1, vx = 1: u = 16 -> fu = 4 = w, rejected
    assert idx["valid"][0, 0, 0, 0, 0] == 0 and cnt[0, 0, 0] == 0 and np.all(out[0, 0, 0] == 0)


def test_behind_camera_and_empty_cells_are_zero():
    feats = np.ones((1, 1, 2, 4, 2), dtype=np.float32)
    depth = np.ones((1, 1, 2, 4, 2), dtype=np.float32)
    p = _one_camera_problem(O.MODE_LAPLACE, depth, feats)
    p.roi = [-4.0, -1.0, -2.0, 2.0, -1.0, 1.0]  # every cell behind the camera
    out, cnt = O.forward(p, with_count=True)
    assert np.all(out == 0) and np.all(cnt == 0)
    df, dd = O.backward(p, np.ones(p.out_shape, np.float32))
    assert np.all(df == 0) and np.all(dd == 0)


@pytest.mark.parametrize("mode", ["laplace", "categorical"])
def test_sum_is_mean_times_count_and_rows_compose(mode):
    inp = inputs_for(SMALL, mode)
    mean, cnt = O.forward(oracle_problem(inp, SMALL, mode, pool="mean"), with_count=True)
    total = O.forward(oracle_problem(inp, SMALL, mode, pool="sum"))
    assert rel_err(mean * cnt[..., None], total) < TOL_F32
    top = O.forward(oracle_problem(inp, SMALL, mode, pool="sum", y_range=(0, 13)))
    bottom = O.forward(oracle_problem(inp, SMALL, mode, pool="sum", y_range=(13, SMALL.Y)))
    assert np.array_equal(top + bottom, total) and np.all(top[:, 13:] == 0) and np.all(bottom[:, :13] == 0)


def test_indices_agree_with_forward_count():
    for mode in ("gaussian", "categorical"):
        inp = inputs_for(SMALL, mode)
        p = oracle_problem(inp, SMALL, mode, threshold=1e-3)
        _, cnt = O.forward(p, with_count=True)
        idx = O.indices(p)
        assert np.array_equal(idx["count"], cnt)
        assert np.array_equal(idx["valid"].sum(axis=(1, 4)).astype(np.int32), cnt)
        assert ((idx["u0"] >= 0) == (idx["valid"] == 1)).all()
        if mode == "categorical":
            assert idx["kbin"][idx["valid"] == 1].min() >= 0 and idx["kbin"].max() < SMALL.D
        else:
            assert (idx["kbin"] == -1).all()


def test_backward_is_the_adjoint_of_forward():
    """<forward(f), g> = <f, d_feats(g)> (linear in the features) and the same for the categorical
    probabilities, evaluated in float64."""
    inp = inputs_for(SMALL, "categorical")
    p = oracle_problem(inp, SMALL, "categorical")
    go = synth.upstream_grad(SMALL).numpy()
    out = O.forward(p, dtype=np.float64)
    d_feats, d_depth = O.backward(p, go, dtype=np.float64)
    lhs = (out * go).sum()
    assert abs(lhs - (p.feats.astype(np.float64) * d_feats).sum()) < 1e-9 * abs(lhs)
    assert abs(lhs - (p.depth.astype(np.float64) * d_depth).sum()) < 1e-9 * abs(lhs)


def test_parametric_depth_gradient_by_finite_differences():
    inp = inputs_for(SMALL, "gaussian")
    p = oracle_problem(inp, SMALL, "gaussian")
    go = synth.upstream_grad(SMALL).numpy()
    _, d_depth = O.backward(p, go, dtype=np.float64)
    rng = np.random.RandomState(0)
    # base and step on a 2^-10 lattice, so that base +- step is exact in float32
    p.depth = np.round(p.depth * 1024.0) / 1024.0
    _, d_depth = O.backward(p, go, dtype=np.float64)
    direction = (rng.randint(-4, 5, size=p.depth.shape) / 512.0).astype(np.float32)
    base = p.depth.copy()
    p.depth = base + direction
    plus = (O.forward(p, dtype=np.float64) * go).sum()
    p.depth = base - direction
    minus = (O.forward(p, dtype=np.float64) * go).sum()
    fd = (plus - minus) / 2.0
    an = (d_depth * direction.astype(np.float64)).sum()
    assert abs(fd - an) < 1e-4 * abs(an)


def test_legacy_depth_gradient_writes_the_same_value_twice():
    inp = inputs_for(SMALL, "laplace")
    p = oracle_problem(inp, SMALL, "laplace")
    _, dd = O.backward(p, synth.upstream_grad(SMALL).numpy(), legacy_depth_grad=True)
    assert np.array_equal(dd[..., 0], dd[..., 1]) and np.abs(dd).max() > 0


def test_threads_do_not_change_the_forward():
    inp = inputs_for(SMALL, "categorical")
    p = oracle_problem(inp, SMALL, "categorical")
    assert np.array_equal(O.forward(p, threads=1), O.forward(p, threads=4))


def test_projection_matrices_match_the_reference_builder():
    """create_projection_matrix (sampling_vt.py:21-33) on a seeded rig; float32 there, float64 here."""
    g = projection_golden()
    P = O.projection(g["sensor2ego"], g["camera2imgs"], g["post_rots"], g["post_trans"])
    per_cam = np.abs(P - g["proj"]).reshape(-1, 12).max(1) / np.abs(g["proj"]).reshape(-1, 12).max(1)
    assert per_cam.max() < 1e-5


def test_projection_host_fallback_matches_the_oracle():
    """The torch branch of flashbev_b200.create_projection_matrix (CPU tensors)."""
    import torch
    from flashbev_b200.sampling_vt import create_projection_matrix
    g = projection_golden()
    t = {k: torch.from_numpy(g[k]) for k in ("sensor2ego", "camera2imgs", "post_rots", "post_trans")}
    P = create_projection_matrix(t["sensor2ego"], None, t["camera2imgs"], t["post_rots"], t["post_trans"], None).numpy()
    ref = O.projection(g["sensor2ego"], g["camera2imgs"], g["post_rots"], g["post_trans"])
    assert np.abs(P - ref).max() / np.abs(ref).max() < 1e-5


def test_projection_rejects_a_singular_pose():
    g = projection_golden()
    s2e = g["sensor2ego"].copy()
    s2e[0, 0, 2] = 0.0  # a zero row: the elimination meets an exact zero pivot
    with pytest.raises(ValueError):
        O.projection(s2e, g["camera2imgs"], g["post_rots"], g["post_trans"])


def test_float32_geometry_rounding_floor_on_the_training_shape():
    """How far ANY float32 evaluation of the operator is from exact arithmetic on the training shape (cfg3: image
    512x1408, feature maps 32x88, one sample here).  Everything is evaluated twice with the same integer decisions
    (texels, acceptance): in the oracle's pinned float32 order, and in float64 from the projection on.  The feature
    coordinate reaches 88, where a float32 ulp is 7.6e-6 of a texel, and the bilinear weights inherit that: the two
    results are about 1.2e-5 apart (max|a-b| / max|b|).  That is the floor below which two float32 implementations
    that round the geometry differently (this library's pinned order, the reference binary's compiler-chosen
    contraction) cannot be compared; the 1e-5 bar therefore applies against the oracle's pinned order, and the
    comparison with the reference's CUDA kernels on this shape uses 3e-5."""
    from flashbev_b200 import synth
    from tests.helpers import host_threads, inputs_for, oracle_problem, rel_err
    w = synth.workload("cfg3", B=1)
    inp = inputs_for(w, "laplace")
    p = oracle_problem(inp, w, "laplace", threshold=1e-6)
    pinned = O.forward(p, threads=host_threads())[0]
    idx = O.indices(p)
    feats = inp["image_feats"].double().numpy()[0]
    depth = inp["depth_params"].double().numpy()[0]
    P = inp["projection_matrices"].double().numpy()[0]
    X, Y, Z = w.grid
    roi = np.array(w.roi, np.float32)
    vs = [np.float64(np.float32((roi[2 * i + 1] - roi[2 * i]) / np.float32(g))) for i, g in enumerate((X, Y, Z))]
    axes = [np.float64(roi[2 * i]) + (np.arange(g) + 0.5) * vs[i] for i, g in enumerate((X, Y, Z))]
    gx, gy, gz = np.meshgrid(*axes, indexing="xy")  # [Y,X,Z]
    ih, iw = w.image_size
    out = np.zeros((Y, X, w.C))
    cnt = np.zeros((Y, X))
    for n in range(w.N):
        u, v, d = (P[n, r, 0] * gx + P[n, r, 1] * gy + P[n, r, 2] * gz + P[n, r, 3] for r in range(3))
        cd = np.maximum(d, 1e-6)
        fu, fv = u / cd / iw * w.W, v / cd / ih * w.H
        valid = idx["valid"][0, n].astype(bool)
        u0, v0 = np.where(valid, idx["u0"][0, n], 0), np.where(valid, idx["v0"][0, n], 0)
        du, dv = fu - u0, fv - v0
        u1, v1 = np.minimum(u0 + 1, w.W - 1), np.minimum(v0 + 1, w.H - 1)
        wts = [((1 - du) * (1 - dv), v0, u0), ((1 - du) * dv, v1, u0), (du * (1 - dv), v0, u1), (du * dv, v1, u1)]
        mean = sum(wt * depth[n, vv, uu, 0] for wt, vv, uu in wts)
        sigma = sum(wt * depth[n, vv, uu, 1] for wt, vv, uu in wts)
        wgt = np.where(valid, 0.5 * np.exp(-np.abs((d - mean) / (sigma + 1e-6))) / (sigma + 1e-6), 0.0)
        for z in range(Z):
            f = sum(wt[..., z, None] * feats[n, vv[..., z], uu[..., z]] for wt, vv, uu in wts)
            out += f * wgt[..., z, None]
        cnt += valid.sum(-1)
    exact = np.where(cnt[..., None] > 0, out / np.maximum(cnt, 1)[..., None], 0.0)
    floor = rel_err(pinned, exact)
    assert 5e-6 < floor < 2e-5, floor
