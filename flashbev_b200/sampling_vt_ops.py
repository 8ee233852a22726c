"""``sampling_vt_pillarpool_fused``: pillar pooling over pre-sorted sample lists, the reference's comparison
baseline (flashbev/flashbevpool/sampling_vt_ops.py:8-32 on src/sampling_vt_cuda.cu:24-148), on libfbev.so.

Same arguments, same result layout: ``out`` is a zero-filled tensor of ``bev_feat_shape`` (channels last) whose
cells with at least one listed sample receive the mean of ``weight x bilinear feature`` over their samples; the
return value is that tensor with the channel axis moved to position 1.  Float32 only, as in the reference; there
is no CPU path.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["sampling_vt_pillarpool_fused"]


def sampling_vt_pillarpool_fused(depth, feat, u_coords, v_coords, z_coords, batch_camera_indices, ranks_bev,
                                 bev_feat_shape, interval_starts, interval_lengths, batch_size, num_cameras, feat_h,
                                 feat_w, epsilon=1e-6, depth_distribution=0):
    if not feat.is_cuda:
        raise RuntimeError("sampling_vt_pillarpool_fused runs on CUDA tensors only (there is no CPU path)")
    dev = feat.device
    f32 = lambda t: t.to(device=dev, dtype=torch.float32).contiguous()  # noqa: E731
    i32 = lambda t: t.to(device=dev, dtype=torch.int32).contiguous()  # noqa: E731
    depth, feat = f32(depth), f32(feat)
    u, v, z = f32(u_coords), f32(v_coords), f32(z_coords)
    cams, ranks = i32(batch_camera_indices), i32(ranks_bev)
    starts, lengths = i32(interval_starts), i32(interval_lengths)
    shape = tuple(int(s) for s in bev_feat_shape)
    out = feat.new_zeros(shape)
    c = feat.shape[-1]
    if shape[-1] != c or depth.shape[-1] != 2:
        raise ValueError(f"feat must be [..., {shape[-1]}] and depth [..., 2]; got {tuple(feat.shape)}, {tuple(depth.shape)}")
    with torch.cuda.device(dev):
        rc = _lib.load().fbev_pillar_pool(
            c, starts.numel(), depth.data_ptr(), feat.data_ptr(), u.data_ptr(), v.data_ptr(), z.data_ptr(),
            cams.data_ptr(), ranks.data_ptr(), starts.data_ptr(), lengths.data_ptr(), int(batch_size), int(num_cameras),
            int(feat_h), int(feat_w), float(epsilon), int(depth_distribution), out.data_ptr(),
            torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "fbev_pillar_pool")
    return out.movedim(-1, 1).contiguous()
