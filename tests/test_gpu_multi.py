"""Two-GPU test of row and batch sharding over NCCL (skipped on a single-GPU box): every rank must end up
with exactly what one GPU computes alone, and the row-sharded backward with the summed partial gradients."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flashbev_b200 import flash_bevpool, sharding, synth
        w = synth.workload("cfg5", X=128, Y=96, Z=8, C=64)
        kw = dict(depth_distribution=2, depth_bin_range=(w.d0, w.delta), depth_weight_threshold=0.0)
        inp = {k: v.to(dev) for k, v in synth.make_inputs(w, "categorical", dtype="fp32").items()}
        go = synth.upstream_grad(w).to(dev)
        # one GPU alone
        f0 = inp["image_feats"].clone().requires_grad_(True)
        d0 = inp["depth_params"].clone().requires_grad_(True)
        alone = flash_bevpool(f0, d0, *[inp[k] for k in ("projection_matrices", "feature_size", "image_size",
                                                          "roi_range", "grid_size")], **kw)
        alone.backward(go)
        # rows over the ranks
        f1 = inp["image_feats"].clone().requires_grad_(True)
        d1 = inp["depth_params"].clone().requires_grad_(True)
        rows = sharding.flash_bevpool_rows(f1, d1, inp["projection_matrices"], inp["feature_size"], inp["image_size"],
                                           inp["roi_range"], inp["grid_size"], **kw)
        rows.backward(go)
        ok_rows = bool(torch.equal(rows, alone))
        # rows over the ranks without a collective: the kernel stores into every rank's buffer
        args = [inp[k] for k in ("projection_matrices", "feature_size", "image_size", "roi_range", "grid_size")]
        ok_p2p = True
        for call in range(3):  # the two symmetric buffers alternate; the third call reuses the first
            scale_in = 1.0 + call
            p2p = sharding.flash_bevpool_rows_p2p(inp["image_feats"] * scale_in, inp["depth_params"], *args, **kw)
            want = flash_bevpool(inp["image_feats"] * scale_in, inp["depth_params"], *args, **kw)
            ok_p2p = ok_p2p and bool(torch.equal(p2p, want))
            mc = sharding.flash_bevpool_rows_p2p(inp["image_feats"] * scale_in, inp["depth_params"], *args, **kw,
                                                 multicast=True)  # falls back to peer stores without NVLS
            ok_p2p = ok_p2p and bool(torch.equal(mc, want))
        # rows kept sharded: this rank's rows equal the same rows of one GPU's output; the input gradients, summed
        # over the ranks, equal one GPU's
        f2 = inp["image_feats"].clone().requires_grad_(True)
        d2 = inp["depth_params"].clone().requires_grad_(True)
        mine = sharding.flash_bevpool_rows_local(f2, d2, *args, **kw)
        ry0, ry1 = sharding.row_slice(w.Y, world, rank)
        ok_p2p = ok_p2p and bool(torch.equal(mine, alone[:, ry0:ry1]))
        mine.backward(go[:, ry0:ry1])
        sharding.all_reduce_input_grads(f2, d2)
        ok_p2p = ok_p2p and float((f2.grad - f0.grad).abs().max()) < 1e-5 * float(f0.grad.abs().max())
        ok_p2p = ok_p2p and float((d2.grad - d0.grad).abs().max()) < 1e-5 * float(d0.grad.abs().max())
        # device time of the two row-split forwards (informative)
        def timed(fn, n=20):
            for _ in range(3):
                fn()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            dist.barrier()
            s.record()
            for _ in range(n):
                fn()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / n * 1e3
        with torch.no_grad():
            t_nccl = timed(lambda: sharding.flash_bevpool_rows(inp["image_feats"], inp["depth_params"], *args, **kw))
            t_p2p = timed(lambda: sharding.flash_bevpool_rows_p2p(inp["image_feats"], inp["depth_params"], *args, **kw))
            t_one = timed(lambda: flash_bevpool(inp["image_feats"], inp["depth_params"], *args, **kw))
        if rank == 0:
            print(f"row split on {world} GPUs: all-gather {t_nccl:.1f} us, peer stores {t_p2p:.1f} us, one GPU {t_one:.1f} us",
                  flush=True)
        scale = float(f0.grad.abs().max())
        ok_gf = float((f1.grad - f0.grad).abs().max()) < 1e-5 * scale
        ok_gd = float((d1.grad - d0.grad).abs().max()) < 1e-5 * float(d0.grad.abs().max())
        # batch over the ranks
        wb = synth.workload("cfg4", B=4)
        whole = {k: v.to(dev) for k, v in synth.make_inputs(wb, "categorical").items()}
        b0, b1 = sharding.batch_slice(wb.B, world, rank)
        part = {k: v.to(dev) for k, v in synth.make_inputs(wb, "categorical", batch_slice=(b0, b1)).items()}
        full = flash_bevpool(**whole, **kw)
        gathered = sharding.flash_bevpool_batch(part["image_feats"], part["depth_params"], part["projection_matrices"],
                                                part["feature_size"], part["image_size"], part["roi_range"],
                                                part["grid_size"], batch=wb.B, gather=True, **kw)
        ok_batch = bool(torch.equal(gathered, full))
        torch.cuda.synchronize()
        results.put((rank, ok_rows and ok_p2p, ok_gf, ok_gd, ok_batch))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_and_batch_sharding_over_nccl():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    got = [results.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok_rows, ok_gf, ok_gd, ok_batch in got:
        assert ok_rows and ok_gf and ok_gd and ok_batch, (rank, ok_rows, ok_gf, ok_gd, ok_batch)
