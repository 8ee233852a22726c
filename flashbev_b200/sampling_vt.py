"""``SamplingVT``: the caller of the fused operator, shaped like the reference module.

Counterpart of flashbev/flashbevpool/sampling_vt.py:126-294.  Constructor arguments,
sub-module names (``context_network``, ``depth_network``: 1x1 convolutions, so reference
state dicts load), buffers and the ``forward(input) -> (bev_features [B,C,Y,X], depths)``
contract are the reference's, which is what tools/utils/transformer_utils.py:26-44 and
tools/profile_differences.py:237 rely on.

  fuse_projection=True   -> the fused CUDA operator (``flash_bevpool``).
  fuse_projection=False, use_bev_pool=False
                         -> a dense PyTorch evaluation of the same sampling (every voxel
                            materialised), the comparison baseline of the reference's
                            harnesses.  Written with explicit gathers; it is a comparison
                            method, not a fallback of the fused path.
  fuse_projection=False, use_bev_pool=True
                         -> the reference's sort-based pillar-pool baseline (sampling_vt.py:296-335,
                            381-447): project every voxel, keep the samples a camera sees, sort them
                            by BEV cell, pool each cell's interval with ``sampling_vt_pillarpool_fused``.
                            A comparison method too.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .flash_bevpool import flash_bevpool
from .sampling_vt_ops import sampling_vt_pillarpool_fused


def create_projection_matrix(sensor2ego, ego2global, camera2imgs, post_rots, post_trans, bda):
    """[B,N,3,4] voxel -> (u*d, v*d, d) matrices from the camera calibration.

    P = [post_rots @ K, with post_trans added to column 2] @ inverse(sensor2ego), rows 0-2
    (sampling_vt.py:21-33).  ``ego2global`` and ``bda`` are accepted and unused, as there.
    """
    B, N = camera2imgs.shape[:2]
    if camera2imgs.is_cuda and all(t.dtype == torch.float32 for t in (sensor2ego, camera2imgs, post_rots, post_trans)):
        # one kernel (fbev_projection_matrices) instead of inverse + matmuls + slicing
        from . import _lib
        dev = camera2imgs.device
        args = [t.expand(B, N, *t.shape[2:]).contiguous() for t in (sensor2ego, camera2imgs, post_rots, post_trans)]
        out = torch.empty(B, N, 3, 4, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.load().fbev_projection_matrices(*[a.data_ptr() for a in args], out.data_ptr(), B * N,
                                                      torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "fbev_projection_matrices")
        return out
    intrinsic = torch.zeros(B, N, 4, 4, device=camera2imgs.device, dtype=camera2imgs.dtype)
    intrinsic[..., 3, 3] = 1.0
    intrinsic[..., :3, :3] = post_rots @ camera2imgs
    intrinsic[..., :3, 2] += post_trans
    return (intrinsic @ torch.linalg.inv(sensor2ego))[:, :, :3, :]


def dense_sampling_vt(features_pv, depths, projection_matrices, image_size, roi_ranges, grid, depth_distribution,
                      depth_weight_threshold, epsilon=1e-6):
    """Dense evaluation: features_pv [B*N,C,h,w], depths [B*N,2,h,w] -> [B,C,Y,X].

    Same sampling rule as the fused kernel (flash_bevpool_cuda.cu:101-216): project every voxel
    centre, reject behind-camera / out-of-map samples, bilinear weights with the last row and
    column clamped, likelihood weight, mean over accepted samples.
    """
    BN, C, h, w = features_pv.shape
    B, N = projection_matrices.shape[:2]
    X, Y, Z = grid
    dev, dt = features_pv.device, torch.float32
    roi = roi_ranges.to(dt)
    axes = []
    for i, g in enumerate((X, Y, Z)):
        vs = (roi[i, 1] - roi[i, 0]) / g
        axes.append(roi[i, 0] + (torch.arange(g, device=dev, dtype=dt) + 0.5) * vs)
    gx, gy, gz = torch.meshgrid(*axes, indexing="ij")
    pts = torch.stack([gx, gy, gz, torch.ones_like(gx)], dim=-1).reshape(-1, 4)          # [V,4]
    uvd = torch.einsum("bnij,vj->bnvi", projection_matrices.to(dt), pts)                  # [B,N,V,3]
    d = uvd[..., 2]
    cd = torch.clamp(d, min=epsilon)
    fu = uvd[..., 0] / cd / image_size[1] * w
    fv = uvd[..., 1] / cd / image_size[0] * h
    ok = (d > 0) & (fu >= 0) & (fu < w) & (fv >= 0) & (fv < h)
    u0 = fu.floor().clamp(0, w - 1)
    v0 = fv.floor().clamp(0, h - 1)
    du, dv = fu - u0, fv - v0
    u0, v0 = u0.long(), v0.long()
    u1, v1 = (u0 + 1).clamp(max=w - 1), (v0 + 1).clamp(max=h - 1)
    wts = [((1 - du) * (1 - dv), v0, u0), ((1 - du) * dv, v1, u0), (du * (1 - dv), v0, u1), (du * dv, v1, u1)]
    feats = features_pv.reshape(B, N, C, h * w).to(dt)
    deps = depths.reshape(B, N, 2, h * w).to(dt)
    V = pts.shape[0]
    f3 = torch.zeros(B, N, C, V, device=dev, dtype=dt)
    p3 = torch.zeros(B, N, 2, V, device=dev, dtype=dt)
    for wt, vv, uu in wts:
        idx = (vv * w + uu).clamp(0, h * w - 1)
        f3 += torch.gather(feats, 3, idx.unsqueeze(2).expand(-1, -1, C, -1)) * wt.unsqueeze(2)
        p3 += torch.gather(deps, 3, idx.unsqueeze(2).expand(-1, -1, 2, -1)) * wt.unsqueeze(2)
    mu, sigma = p3[:, :, 0], p3[:, :, 1]
    zs = (d - mu) / (sigma + epsilon)
    if depth_distribution == "laplace":
        prob = 0.5 * torch.exp(-zs.abs()) / (sigma + epsilon)
    else:
        prob = torch.exp(-0.5 * zs * zs) / (sigma + epsilon)
    ok = ok & ~(prob < depth_weight_threshold)
    contrib = torch.where(ok.unsqueeze(2), f3 * prob.unsqueeze(2), torch.zeros((), device=dev, dtype=dt))
    bev = contrib.reshape(B, N, C, X, Y, Z).sum(dim=(1, 5))                               # [B,C,X,Y]
    cnt = ok.reshape(B, N, X, Y, Z).sum(dim=(1, 4)).clamp(min=1).to(dt)
    return (bev / cnt.unsqueeze(1)).transpose(-1, -2).contiguous()                        # [B,C,Y,X]


def project_voxels(projection_matrices, grid_axes, epsilon=1e-6):
    """(u, v, d) of every voxel centre in every camera: [B,N,X,Y,Z] each (sampling_vt.py:449-466).
    ``grid_axes``: the three 1-D tensors of voxel-centre coordinates."""
    ax, ay, az = grid_axes
    P = projection_matrices.to(ax.dtype)
    # P[..., 0:3] . (x, y, z) + P[..., 3], axis by axis: no [V,4] point tensor is formed
    px = P[..., 0].unsqueeze(-1) * ax          # [B,N,3,X]
    py = P[..., 1].unsqueeze(-1) * ay          # [B,N,3,Y]
    pz = P[..., 2].unsqueeze(-1) * az          # [B,N,3,Z]
    uvd = (px[..., :, None, None] + py[..., None, :, None] + pz[..., None, None, :] +
           P[..., 3][..., None, None, None])  # [B,N,3,X,Y,Z]
    d = uvd[:, :, 2]
    cd = torch.where(d >= 0, d.clamp(min=epsilon), d.clamp(max=-epsilon))
    return uvd[:, :, 0] / cd, uvd[:, :, 1] / cd, d


def pillar_pool_lists(u, v, d, image_size, feature_size):
    """Sample lists of the pillar-pool baseline (sampling_vt.py:296-361): the (b, n, x, y, z) samples that fall inside
    their camera's feature map with positive depth, ordered by BEV cell (b, x, y), and one interval per cell that
    has any.  Returns feature-map coordinates u, v, depth, camera index b * N + n, cell rank, interval starts and
    lengths."""
    B, N, X, Y, Z = d.shape
    fh, fw = feature_size
    fu = u / image_size[1] * fw
    fv = v / image_size[0] * fh
    inside = (fu >= 0) & (fu < fw) & (fv >= 0) & (fv < fh) & (d > 0)
    b, n, x, y, _ = inside.nonzero(as_tuple=True)       # row-major: camera-major, height-minor within a cell
    rank = (b * X + x) * Y + y
    rank, order = torch.sort(rank, stable=True)
    cells, lengths = torch.unique_consecutive(rank, return_counts=True)
    starts = torch.cumsum(lengths, 0) - lengths
    pick = lambda t: t[inside][order]  # noqa: E731
    return pick(fu), pick(fv), pick(d), (b * N + n)[order], rank, starts, lengths


class SamplingVT(nn.Module):
    """View transformer: 1x1 context / depth heads followed by BEV pooling (sampling_vt.py:126-234)."""

    def __init__(self, grid_config, input_size, downsample=16, in_channels=512, out_channels=64,
                 fuse_projection=True, use_bev_pool=True, use_shared_memory=False, fuse_bilinear=False,
                 depth_distribution="laplace", optimize_z_precompute=True, use_warp_kernel=False,
                 use_vectorized_load=False, depth_weight_threshold=0.0):
        super().__init__()
        self.use_bev_pool = use_bev_pool
        self.out_channels = out_channels
        self.in_channels = in_channels
        self.image_size = input_size
        self.depth_range = grid_config["depth"][:2]
        self.use_shared_memory = use_shared_memory
        self.fuse_projection = fuse_projection
        self.fuse_bilinear = fuse_bilinear
        self.optimize_z_precompute = optimize_z_precompute
        self.use_warp_kernel = use_warp_kernel
        self.use_vectorized_load = use_vectorized_load
        self.depth_weight_threshold = depth_weight_threshold
        self.depth_distribution = depth_distribution.lower()
        if self.depth_distribution not in ("laplace", "gaussian"):
            raise ValueError(f"depth_distribution must be 'laplace' or 'gaussian', got '{depth_distribution}'")
        self.context_network = nn.Conv2d(in_channels, out_channels, kernel_size=1, padding=0)
        self.register_buffer("depth_bins", torch.arange(*grid_config["depth"], dtype=torch.float))
        self.num_depth_bins = len(self.depth_bins)
        self.depth_network = nn.Sequential(nn.Conv2d(in_channels, 2, kernel_size=1, padding=0), nn.ReLU())
        axes = [grid_config["x"], grid_config["y"], grid_config["z"]]
        self.register_buffer("roi_ranges", torch.as_tensor([a[:2] for a in axes]))
        self.register_buffer("output_grid_size", torch.tensor(
            [(axes[0][1] - axes[0][0]) / axes[0][2], (axes[1][1] - axes[1][0]) / axes[1][2], 1], dtype=torch.int32))
        self.register_buffer("sample_grid_size", torch.tensor(
            [(a[1] - a[0]) / a[2] for a in axes], dtype=torch.int32))
        self._grid = tuple(int(v) for v in self.sample_grid_size.tolist())
        if not fuse_projection:
            # buffers of the reference's unfused branches (sampling_vt.py:187-196), so that its state dicts load
            self.register_buffer("voxel_size", torch.as_tensor([a[2] for a in axes]))
            centres = [torch.linspace(a[0], a[1], g + 1)[:-1] + a[2] / 2.0 for a, g in zip(axes, self._grid)]
            self.register_buffer("coords_3d", torch.stack(torch.meshgrid(*centres, indexing="ij"), dim=-1))
        # small constant inputs of the operator, built once per (device, B, N, h, w)
        self._const_cache = {}

    @staticmethod
    def _pointwise_conv(conv, x):
        """1x1 convolution of x [BN,C,H,W] whose result is laid out [BN,H,W,O] in memory and returned as the
        [BN,O,H,W] view of it (channels-last strides).  The operator wants channels-last features; the
        reference converts with movedim + contiguous after the convolution (sampling_vt.py:252-253).  Here
        the batched GEMM takes x as a transposed operand, so no transpose kernel runs on either side."""
        BN, C, H, W = x.shape
        O = conv.out_channels
        if x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous():
            xm = x.permute(0, 2, 3, 1).reshape(BN, H * W, C)
        else:
            xm = x.flatten(2).transpose(1, 2)
        wt = conv.weight.view(O, C).t().unsqueeze(0).expand(BN, C, O)
        bias = conv.bias.view(1, 1, O) if conv.bias is not None else xm.new_zeros(1, 1, O)
        return torch.baddbmm(bias, xm, wt).view(BN, H, W, O).permute(0, 3, 1, 2)

    def forward_depth(self, x):
        depth_params = torch.relu(self._pointwise_conv(self.depth_network[0], x))
        # sigma + 0.1 keeps it away from zero (sampling_vt.py:220-223); out of place, so that the ReLU output
        # autograd saved stays intact and the module can be trained
        return depth_params + depth_params.new_tensor([0.0, 0.1]).view(1, 2, 1, 1)

    def forward(self, input, images=None, img_meta=None, lidar_cloud=None, depth_from_lidar=None):
        x = input[0]
        B, N, C, H, W = x.shape
        x = x.view(B * N, C, H, W)
        features_pv = self._pointwise_conv(self.context_network, x)
        depths = self.forward_depth(x)
        # [B,C,Y,X] with channels-last strides: a channels-last BEV encoder consumes it without a copy
        return self.sampling_vt(input, features_pv, depths), depths

    def _constants(self, device, B, N, h, w):
        key = (str(device), B, N, h, w)
        c = self._const_cache.get(key)
        if c is None:
            c = (torch.tensor([h, w], device=device, dtype=torch.int32).view(1, 1, 2).expand(B, N, -1).contiguous(),
                 torch.tensor([self.image_size[0], self.image_size[1]], device=device, dtype=torch.int32),
                 torch.tensor(self._grid, dtype=torch.int32))  # host tensor: sizes without a device round trip
            self._const_cache[key] = c
        return c

    def sampling_vt(self, input, features_pv, depths):
        B, N = input[3].shape[:2]
        projection_matrices = create_projection_matrix(*input[1:7])
        h, w = features_pv.shape[-2:]
        if self.fuse_projection:
            feature_size, image_size, grid_size = self._constants(features_pv.device, B, N, h, w)
            bev = flash_bevpool(
                image_feats=features_pv.movedim(-3, -1).unflatten(0, (B, N)),
                depth_params=depths.movedim(-3, -1).unflatten(0, (B, N)),
                projection_matrices=projection_matrices,
                depth_distribution=1 if self.depth_distribution == "laplace" else 0,
                use_shared_memory=self.use_shared_memory,
                optimize_z_precompute=self.optimize_z_precompute,
                use_warp_kernel=self.use_warp_kernel,
                use_vectorized_load=self.use_vectorized_load,
                feature_size=feature_size,
                image_size=image_size,
                roi_range=self.roi_ranges.flatten(),
                grid_size=grid_size,
                epsilon=1e-6,
                depth_weight_threshold=self.depth_weight_threshold,
            )
            return bev.movedim(-1, -3)
        if self.use_bev_pool:
            c3 = self.coords_3d
            u, v, d = project_voxels(projection_matrices, (c3[:, 0, 0, 0], c3[0, :, 0, 1], c3[0, 0, :, 2]))
            fu, fv, fd, cams, ranks, starts, lengths = pillar_pool_lists(u, v, d, self.image_size, (h, w))
            X, Y = self._grid[0], self._grid[1]
            bev = sampling_vt_pillarpool_fused(
                depth=depths.movedim(-3, -1), feat=features_pv.movedim(-3, -1), u_coords=fu, v_coords=fv, z_coords=fd,
                batch_camera_indices=cams, ranks_bev=ranks, bev_feat_shape=(B, X, Y, 1, features_pv.shape[-3]),
                interval_starts=starts, interval_lengths=lengths, batch_size=B, num_cameras=N, feat_h=h, feat_w=w,
                epsilon=1e-6, depth_distribution=1 if self.depth_distribution == "laplace" else 0)
            return bev.squeeze(-1).movedim(-1, -2)   # [B,C,X,Y,1] -> [B,C,Y,X]
        return dense_sampling_vt(features_pv, depths, projection_matrices, self.image_size, self.roi_ranges,
                                 self._grid, self.depth_distribution, self.depth_weight_threshold)
