"""CPU tests of the multi-GPU plumbing with two gloo ranks.  The per-rank compute is a stand-in built
on the CPU oracle (tests may use it; the product path never does): what is checked here is the
slicing, the all-gather of rows / batch slices and the all-reduce of the partial gradients."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashbev_b200 import sharding, synth
from oracle import oracle as O
from tests.helpers import SMALL, inputs_for, oracle_problem


def test_even_slices_cover_everything_once():
    for n in (1, 7, 64, 200, 513):
        for world in (1, 2, 3, 8):
            cuts = [sharding.even_slice(n, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [b - a for a, b in cuts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.even_slice(4, 2, 2)


class OraclePool(torch.autograd.Function):
    """CPU stand-in of the operator (categorical depth, sum pooling) with y_range support."""

    @staticmethod
    def forward(ctx, feats, depth, proj, fs, isz, roi, grid, y_range):
        w = SMALL
        inp = dict(image_feats=feats.detach(), depth_params=depth.detach(), projection_matrices=proj, feature_size=fs,
                   image_size=isz, roi_range=roi, grid_size=grid)
        ctx.problem = oracle_problem(inp, w, "categorical", y_range=y_range)
        return torch.from_numpy(O.forward(ctx.problem))

    @staticmethod
    def backward(ctx, go):
        df, dd = O.backward(ctx.problem, go.numpy())
        return torch.from_numpy(df), torch.from_numpy(dd), None, None, None, None, None, None


def oracle_op(feats, depth, proj, fs, isz, roi, grid, y_range=None, **_):
    return OraclePool.apply(feats, depth, proj, fs, isz, roi, grid, y_range)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = SMALL
        inp = inputs_for(w, "categorical")
        # ---- rows split over the ranks, forward + backward ----
        f = inp["image_feats"].clone().requires_grad_(True)
        d = inp["depth_params"].clone().requires_grad_(True)
        out = sharding.flash_bevpool_rows(f, d, inp["projection_matrices"], inp["feature_size"], inp["image_size"],
                                          inp["roi_range"], inp["grid_size"], local_op=oracle_op)
        go = synth.upstream_grad(w)
        out.backward(go)
        # ---- rows that stay sharded: this rank's rows only, gradients of the replicated inputs summed afterwards ----
        f2 = inp["image_feats"].clone().requires_grad_(True)
        d2 = inp["depth_params"].clone().requires_grad_(True)
        mine = sharding.flash_bevpool_rows_local(f2, d2, inp["projection_matrices"], inp["feature_size"],
                                                 inp["image_size"], inp["roi_range"], inp["grid_size"], local_op=oracle_op)
        ry0, ry1 = sharding.row_slice(w.Y, world, rank)
        local_ok = bool(torch.equal(mine, out.detach()[:, ry0:ry1]))
        mine.backward(go[:, ry0:ry1])
        sharding.all_reduce_input_grads(f2, d2)
        local_ok = local_ok and bool(torch.allclose(f2.grad, f.grad, rtol=0, atol=1e-5 * float(f.grad.abs().max())))
        local_ok = local_ok and bool(torch.allclose(d2.grad, d.grad, rtol=0, atol=1e-5 * float(d.grad.abs().max())))
        # ---- batch split over the ranks, gathered ----
        b0, b1 = sharding.batch_slice(w.B, world, rank)
        part = synth.make_inputs(w, "categorical", batch_slice=(b0, b1))
        whole = sharding.flash_bevpool_batch(part["image_feats"], part["depth_params"], part["projection_matrices"],
                                             part["feature_size"], part["image_size"], part["roi_range"],
                                             part["grid_size"], batch=w.B, gather=True, local_op=oracle_op)
        # ---- ragged row shards with B > 1 (36 rows over 2 ranks is even; 35 is not) ----
        rows = torch.arange(2 * 35 * 3 * 2, dtype=torch.float32).view(2, 35, 3, 2)
        y0, y1 = sharding.row_slice(35, world, rank)
        ragged = sharding.gather_rows(rows[:, y0:y1].contiguous(), 35)
        if rank == 0:
            results.put((out.detach().numpy(), f.grad.numpy(), d.grad.numpy(), whole.numpy(),
                         bool(torch.equal(ragged, rows)) and local_ok))
    finally:
        dist.destroy_process_group()


def test_row_and_batch_sharding_with_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    out, gf, gd, whole, ragged_ok = results.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w = SMALL
    inp = inputs_for(w, "categorical")
    p = oracle_problem(inp, w, "categorical")
    ref = O.forward(p)
    rf, rd = O.backward(p, synth.upstream_grad(w).numpy())
    assert np.array_equal(out, ref)                      # rows are computed independently: exact
    assert np.array_equal(whole, ref)                    # so are batch samples
    assert np.allclose(gf, rf, rtol=0, atol=1e-5 * np.abs(rf).max())   # sums of two partial gradients
    assert np.allclose(gd, rd, rtol=0, atol=1e-5 * np.abs(rd).max())
    assert ragged_ok
