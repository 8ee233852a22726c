"""Multi-GPU use of the operator: one process per GPU, ``torch.distributed`` for the plumbing.

The reference has no distributed code.  The operator shards in two ways:

* **batch**: every index of the kernels is prefixed by the batch sample
  (flash_bevpool_cuda.cu:40,57,144), so ranks take contiguous slices of the batch and nothing
  crosses GPUs on the data path.  ``gather=True`` assembles the whole output with one
  ``all_gather_into_tensor`` when a caller needs it on every rank.
* **BEV rows** (one sample, large grid): output rows are independent too.  Rank r computes rows
  ``row_slice(Y, world, r)`` of ``[B, Y, X, C]`` through the operator's ``y_range`` and the rows are
  exchanged with one all-gather.  Inputs are replicated.  In the backward every rank owns the rows
  of the upstream gradient it produced and holds *partial* gradients of the replicated inputs,
  which are summed with one all-reduce each.

Collectives are NCCL's (NVLink / NVSwitch); tensors are in local HBM before any kernel reads them.
``flash_bevpool_rows_p2p`` is the inference form of the row split without a collective: the forward kernel
stores its rows into every rank's output buffer itself (peer stores over NVLink, symmetric memory from
``torch.distributed._symmetric_memory``), and one cross-rank barrier replaces the all-gather.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

import ctypes

from . import _lib
from .flash_bevpool import DepthSpec, _host_values, flash_bevpool, make_problem


def even_slice(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) share of ``n`` items for ``rank``; the first ``n % world`` ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def batch_slice(batch: int, world: int, rank: int) -> Tuple[int, int]:
    return even_slice(batch, world, rank)


ROW_ALIGN = 4  # rows of one tile of the forward kernel


def row_slice(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows of ``rank``: an even share of the rows of tiles, so that every rank works on whole tiles of the
    single-GPU launch and the assembled result is bit-identical to it (the kernel's summation grouping depends on
    the tiling)."""
    t0, t1 = even_slice(-(-rows // ROW_ALIGN), world, rank)
    return min(t0 * ROW_ALIGN, rows), min(t1 * ROW_ALIGN, rows)


def _world(group) -> Tuple[int, int]:
    if not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def gather_batch(local_out: torch.Tensor, batch: int, group=None) -> torch.Tensor:
    """All ranks' batch slices -> the whole ``[batch, Y, X, C]`` tensor on every rank."""
    world, rank = _world(group)
    if world == 1:
        return local_out
    per = -(-batch // world)  # slices are padded to the largest one so that one collective suffices
    pad = local_out.new_zeros((per,) + tuple(local_out.shape[1:]))
    pad[: local_out.shape[0]] = local_out
    full = local_out.new_empty((world * per,) + tuple(local_out.shape[1:]))
    dist.all_gather_into_tensor(full, pad, group=group)
    parts = []
    for r in range(world):
        b0, b1 = batch_slice(batch, world, r)
        parts.append(full[r * per: r * per + (b1 - b0)])
    return torch.cat(parts, dim=0)


def gather_rows(local_rows: torch.Tensor, rows: int, group=None) -> torch.Tensor:
    """Row shards ``[B, rows_r, X, C]`` of every rank -> ``[B, rows, X, C]`` on every rank.

    With B = 1 and ``rows`` divisible by the world size the gathered buffer already is the result;
    otherwise shards are padded to the largest one and stitched together."""
    world, rank = _world(group)
    if world == 1:
        return local_rows
    B = local_rows.shape[0]
    sizes = [y1 - y0 for y0, y1 in (row_slice(rows, world, r) for r in range(world))]
    per = max(sizes)
    if B == 1 and min(sizes) == per:
        full = local_rows.new_empty((1, rows) + tuple(local_rows.shape[2:]))
        dist.all_gather_into_tensor(full.view((rows,) + tuple(local_rows.shape[2:])),
                                    local_rows.reshape((per,) + tuple(local_rows.shape[2:])).contiguous(), group=group)
        return full
    pad = local_rows.new_zeros((B, per) + tuple(local_rows.shape[2:]))
    pad[:, : local_rows.shape[1]] = local_rows
    full = local_rows.new_empty((world * B, per) + tuple(local_rows.shape[2:]))  # rank-major along dim 0
    dist.all_gather_into_tensor(full, pad, group=group)
    full = full.view((world, B, per) + tuple(local_rows.shape[2:]))
    parts = []
    for r in range(world):
        y0, y1 = row_slice(rows, world, r)
        parts.append(full[r, :, : y1 - y0])
    return torch.cat(parts, dim=1)


class _RowShardedPool(torch.autograd.Function):
    """Row-sharded operator with the all-gather in the forward and the gradient all-reduce in the backward."""

    @staticmethod
    def forward(ctx, image_feats, depth_params, local_fn, rows, group):
        world, rank = _world(group)
        y0, y1 = row_slice(rows, world, rank)
        with torch.enable_grad():
            f = image_feats.detach().requires_grad_(image_feats.requires_grad)
            d = depth_params.detach().requires_grad_(depth_params.requires_grad)
            local = local_fn(f, d, (y0, y1))  # [B, Y, X, C] with only rows y0:y1 filled
        ctx.local, ctx.f, ctx.d, ctx.range, ctx.group = local, f, d, (y0, y1), group
        return gather_rows(local[:, y0:y1].contiguous(), rows, group)

    @staticmethod
    def backward(ctx, grad_out):
        y0, y1 = ctx.range
        mine = torch.zeros_like(ctx.local)
        mine[:, y0:y1] = grad_out[:, y0:y1]  # rows this rank produced; the other rows belong to other ranks
        wanted = [t for t in (ctx.f, ctx.d) if t.requires_grad]
        grads = torch.autograd.grad(ctx.local, wanted, mine, allow_unused=True) if wanted else ()
        out = []
        it = iter(grads)
        for t in (ctx.f, ctx.d):
            if not t.requires_grad:
                out.append(None)
                continue
            g = next(it)
            g = torch.zeros_like(t) if g is None else g.contiguous()
            if _world(ctx.group)[0] > 1:
                dist.all_reduce(g, group=ctx.group)  # partial gradients of the replicated inputs
            out.append(g)
        return out[0], out[1], None, None, None


def flash_bevpool_rows_local(image_feats, depth_params, projection_matrices, feature_size, image_size, roi_range,
                             grid_size, group=None, local_op: Optional[Callable] = None, **op_kwargs) -> torch.Tensor:
    """Row split whose result stays split: this rank's rows ``[B, rows_r, X, C]`` (``row_slice``), nothing
    exchanged in the forward.  For a consumer that is sharded by rows too (a BEV encoder with halo exchange, a
    per-region head).  Differentiable; the gradients of the replicated inputs it yields are this rank's partial
    sums, which ``all_reduce_input_grads`` completes.  ``local_op`` replaces ``flash_bevpool`` as the per-rank
    compute (CPU tests of the plumbing)."""
    world, rank = _world(group)
    rows = int(_host_values(grid_size)[1])
    y0, y1 = row_slice(rows, world, rank)
    if local_op is not None:
        return local_op(image_feats, depth_params, projection_matrices, feature_size, image_size, roi_range, grid_size,
                        y_range=(y0, y1), **op_kwargs)[:, y0:y1]
    return flash_bevpool(image_feats, depth_params, projection_matrices, feature_size, image_size, roi_range, grid_size,
                         y_range=(y0, y1), compact_rows=True, **op_kwargs)


def all_reduce_input_grads(*tensors, group=None) -> None:
    """Sums the ``.grad`` of replicated inputs over the ranks (one all-reduce each), after a backward through
    ``flash_bevpool_rows_local``."""
    if _world(group)[0] == 1:
        return
    for t in tensors:
        if t is not None and t.grad is not None:
            dist.all_reduce(t.grad, group=group)


def flash_bevpool_rows(image_feats, depth_params, projection_matrices, feature_size, image_size, roi_range, grid_size,
                       group=None, local_op: Optional[Callable] = None, **op_kwargs) -> torch.Tensor:
    """The operator with its BEV rows split over the ranks of ``group``; returns the whole output on every rank.

    ``image_feats`` / ``depth_params`` are replicated on all ranks.  ``local_op`` replaces ``flash_bevpool`` as
    the per-rank compute (used by CPU tests of the plumbing); it is called as
    ``local_op(image_feats, depth_params, ..., y_range=(y0, y1), **op_kwargs)``.
    """
    op = flash_bevpool if local_op is None else local_op
    rows = int(_host_values(grid_size)[1])

    def local_fn(f, d, y_range):
        return op(f, d, projection_matrices, feature_size, image_size, roi_range, grid_size, y_range=y_range,
                  **op_kwargs)

    return _RowShardedPool.apply(image_feats, depth_params, local_fn, rows, group)


def flash_bevpool_batch(image_feats, depth_params, projection_matrices, feature_size, image_size, roi_range,
                        grid_size, batch: Optional[int] = None, gather: bool = False, group=None,
                        local_op: Optional[Callable] = None, **op_kwargs) -> torch.Tensor:
    """The operator on this rank's slice of the batch (the tensors passed in ARE the slice).

    Nothing is exchanged unless ``gather=True``, which returns the whole ``[batch, Y, X, C]`` output on every
    rank (``batch`` = size of the whole batch; not differentiable through the gather)."""
    op = flash_bevpool if local_op is None else local_op
    out = op(image_feats, depth_params, projection_matrices, feature_size, image_size, roi_range, grid_size,
             **op_kwargs)
    if not gather:
        return out
    if batch is None:
        raise ValueError("gather=True needs the size of the whole batch")
    return gather_batch(out.detach(), batch, group)


# symmetric output buffers per (group, shape, dtype, device): allocation and rendezvous are collective and cost
# milliseconds, the steady state reuses them.  Two buffers alternate, see flash_bevpool_rows_p2p.
_p2p_buffers = {}


def _p2p_buffer(shape, dtype, device, group):
    import torch.distributed._symmetric_memory as symm_mem
    pg = dist.group.WORLD if group is None else group
    key = (pg.group_name, tuple(shape), dtype, str(device))
    hit = _p2p_buffers.get(key)
    if hit is None:
        bufs = [symm_mem.empty(*shape, dtype=dtype, device=device) for _ in range(2)]
        hdls = [symm_mem.rendezvous(b, pg) for b in bufs]
        hit = {"bufs": bufs, "hdls": hdls, "calls": 0, "flag": torch.zeros(1, dtype=torch.int32, device=device)}
        _p2p_buffers[key] = hit
    return hit


def flash_bevpool_rows_p2p(image_feats, depth_params, projection_matrices, feature_size, image_size, roi_range,
                           grid_size, depth_distribution=0, epsilon=1e-6, depth_weight_threshold=1e-6, group=None,
                           multicast=False, **spec_kwargs) -> torch.Tensor:
    """Row-split forward whose kernel writes every rank's copy of the output (inference; no autograd).

    Rank r computes rows ``row_slice(Y, world, r)`` and stores them into its own and all peers' output buffers
    (``fbev_forward_peers``: plain peer stores over NVLink, the kernel waits on nothing).  One tiny NCCL
    all-reduce after the launch is the barrier: when it completes on a rank, every rank's kernel has finished
    and all rows are in this rank's buffer.  It replaces the all-gather of the whole output.

    ``multicast=True`` sends every 16-byte piece once, to the multicast address of the symmetric buffer
    (``fbev_forward_multicast``: the NVSwitch replicates it to all ranks), instead of once per peer; it falls
    back to peer stores where the buffer has no multicast address.

    Two symmetric buffers alternate between calls.  A rank passes the barrier of call k+1 only after every
    rank's stream has finished everything queued before it, the consumers of result k included, so call k+2
    may overwrite the buffer of call k without a second barrier.  The returned tensor is therefore valid until
    the call after the next one with the same shape on this group; consumers must be queued on the calling
    stream (or copy the result).
    """
    world, rank = _world(group)
    if world == 1:
        return flash_bevpool(image_feats, depth_params, projection_matrices, feature_size, image_size, roi_range,
                             grid_size, depth_distribution, epsilon=epsilon,
                             depth_weight_threshold=depth_weight_threshold, **spec_kwargs)
    if world > 8:
        raise ValueError("flash_bevpool_rows_p2p supports up to 8 ranks (one NVLink domain)")
    rows = int(_host_values(grid_size)[1])
    spec = DepthSpec(depth_distribution, y_range=row_slice(rows, world, rank), **spec_kwargs)
    with torch.no_grad():
        p, keep = make_problem(depth_params, image_feats, projection_matrices, feature_size, image_size, roi_range,
                               grid_size, spec, epsilon, depth_weight_threshold)
        feats = keep[0]
        dtype = torch.float32 if spec.out_dtype == torch.float32 else feats.dtype
        state = _p2p_buffer((p.B, p.Y, p.X, p.C), dtype, feats.device, group)
        which = state["calls"] & 1
        state["calls"] += 1
        out, hdl = state["bufs"][which], state["hdls"][which]
        peers = [ptr for r, ptr in enumerate(hdl.buffer_ptrs) if r != rank]
        arr = (ctypes.c_void_p * len(peers))(*peers)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0) if multicast else 0
        with torch.cuda.device(feats.device):
            stream = torch.cuda.current_stream().cuda_stream
            if mc:
                rc = _lib.load().fbev_forward_multicast(ctypes.byref(p), out.data_ptr(), mc, None, stream)
                _lib.check(rc, "fbev_forward_multicast")
            else:
                rc = _lib.load().fbev_forward_peers(ctypes.byref(p), out.data_ptr(), arr, len(peers), None, stream)
                _lib.check(rc, "fbev_forward_peers")
            dist.all_reduce(state["flag"], group=group)  # barrier in stream order
    return out
