"""GPU tests of the caller-side module: ``SamplingVT`` with the fused operator against its dense PyTorch
branch (the comparison the reference's tools/profile_differences.py makes), and the drop-in package name."""
import numpy as np
import pytest
import torch

from flashbev_b200 import synth
from tests.helpers import rel_err

pytestmark = pytest.mark.gpu

GRID = {"x": [-20.0, 20.0, 1.0], "y": [-16.0, 16.0, 1.0], "z": [-4.0, 2.0, 1.0], "depth": [1.0, 60.0, 1.0]}


def _module_inputs(device, B=2, N=6, C=32, H=8, W=22):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B, N, C, H, W, generator=g)
    image = (16 * H, 16 * W)
    P = torch.stack([torch.from_numpy(synth.rig_projection(image, N, jitter_seed=100 + b)) for b in range(B)])
    # sensor2ego / intrinsics that reproduce P: K = I-like split is not needed, feed P through identity parts
    K = torch.eye(3).repeat(B, N, 1, 1)
    s2e = torch.eye(4).repeat(B, N, 1, 1)
    # P = [K|0] @ inv(s2e)  with K = P[:, :, :, :3] and translation folded: solve s2e from P is overkill; instead
    # use the rig's own pieces: f, cx, cy and the camera poses
    import math
    f, cx, cy = 0.35 * image[1], image[1] / 2.0, image[0] / 2.0
    K[:, :, 0, 0] = f
    K[:, :, 1, 1] = f
    K[:, :, 0, 2] = cx
    K[:, :, 1, 2] = cy
    for n in range(N):
        yaw = math.radians(synth.YAWS_DEG[n])
        s2e[:, n, :3, 0] = torch.tensor([math.sin(yaw), -math.cos(yaw), 0.0])
        s2e[:, n, :3, 1] = torch.tensor([0.0, 0.0, -1.0])
        s2e[:, n, :3, 2] = torch.tensor([math.cos(yaw), math.sin(yaw), 0.0])
        s2e[:, n, :3, 3] = torch.tensor([0.8 * math.cos(yaw), 0.8 * math.sin(yaw), 1.5])
    inputs = [x, s2e, torch.eye(4).repeat(B, N, 1, 1), K, torch.eye(3).repeat(B, N, 1, 1), torch.zeros(B, N, 3),
              torch.eye(4).repeat(B, 1, 1)]
    return [t.to(device) for t in inputs], image


@pytest.mark.parametrize("dist", ["laplace", "gaussian"])
def test_sampling_vt_fused_matches_dense_branch(cuda_device, dist):
    from flashbevpool import SamplingVT  # the reference's package name
    inputs, image = _module_inputs(cuda_device)
    outs = []
    for fuse in (False, True):
        torch.manual_seed(42)  # same 1x1 convolutions in both modules (tools/profile_differences.py:218)
        m = SamplingVT(GRID, image, downsample=16, in_channels=32, out_channels=16, fuse_projection=fuse,
                       use_bev_pool=False, depth_distribution=dist, depth_weight_threshold=0.0).to(cuda_device).eval()
        with torch.no_grad():
            bev, depths = m(inputs)
        assert bev.shape == (2, 16, 32, 40) and depths.shape == (12, 2, 8, 22)
        outs.append(bev.float().cpu().numpy())
    dense, fused = outs
    assert rel_err(fused, dense) < 5e-5
    diff = fused.astype(np.float64) - dense
    assert (diff ** 2).mean() < 1e-6 and np.abs(diff).mean() < 1e-6  # tools/profile_differences.py:75-77
    cos = (fused * dense).sum() / (np.linalg.norm(fused) * np.linalg.norm(dense))
    assert cos > 0.9999


def test_sampling_vt_trains_through_the_fused_operator(cuda_device):
    from flashbev_b200 import SamplingVT
    inputs, image = _module_inputs(cuda_device)
    torch.manual_seed(1)
    m = SamplingVT(GRID, image, in_channels=32, out_channels=16, fuse_projection=True, use_bev_pool=False).to(cuda_device)
    bev, _ = m(inputs)
    bev.square().mean().backward()
    grads = [p.grad for p in m.parameters()]
    assert all(g is not None and torch.isfinite(g).all() for g in grads)
    assert sum(float(g.abs().sum()) for g in grads) > 0


@pytest.mark.skipif(False, reason="")
def test_reference_state_dict_names():
    from flashbev_b200 import SamplingVT
    m = SamplingVT(GRID, (128, 352), in_channels=8, out_channels=4, fuse_projection=True, use_bev_pool=False)
    assert {"context_network.weight", "context_network.bias", "depth_network.0.weight", "depth_network.0.bias",
            "depth_bins", "roi_ranges", "output_grid_size", "sample_grid_size"} <= set(m.state_dict().keys())


def test_projection_kernel_matches_oracle_and_reference_builder(cuda_device):
    """fbev_projection_matrices against the float64 oracle and the reference's float32 builder output."""
    from oracle import oracle as O
    from flashbev_b200.sampling_vt import create_projection_matrix
    from tests.helpers import projection_golden
    g = projection_golden()
    t = {k: torch.from_numpy(g[k]).to(cuda_device) for k in ("sensor2ego", "camera2imgs", "post_rots", "post_trans")}
    P = create_projection_matrix(t["sensor2ego"], None, t["camera2imgs"], t["post_rots"], t["post_trans"], None)
    assert P.shape == (3, 6, 3, 4) and P.dtype == torch.float32 and P.is_cuda
    P = P.cpu().numpy().astype(np.float64)
    ref = O.projection(g["sensor2ego"], g["camera2imgs"], g["post_rots"], g["post_trans"])
    scale = np.abs(ref).reshape(-1, 12).max(1)
    # float32 rounding of the result only: half an ulp of the largest entry per camera
    assert (np.abs(P - ref).reshape(-1, 12).max(1) / scale).max() < 1.2e-7
    assert (np.abs(P - g["proj"]).reshape(-1, 12).max(1) / scale).max() < 1e-5


def test_projection_kernel_accepts_broadcast_views(cuda_device):
    """Expanded (stride-0) calibration tensors are materialised before the launch."""
    from oracle import oracle as O
    from flashbev_b200.sampling_vt import create_projection_matrix
    from tests.helpers import projection_golden
    g = projection_golden()
    one = {k: torch.from_numpy(g[k][:1, :1]).to(cuda_device) for k in ("sensor2ego", "camera2imgs", "post_rots", "post_trans")}
    cams = torch.from_numpy(g["camera2imgs"][:1]).to(cuda_device)
    P = create_projection_matrix(one["sensor2ego"].expand(1, 6, 4, 4), None, cams, one["post_rots"].expand(1, 6, 3, 3),
                                 one["post_trans"].expand(1, 6, 3), None).cpu().numpy().astype(np.float64)
    rep = lambda k: np.repeat(g[k][:1, :1], 6, axis=1)  # noqa: E731
    ref = O.projection(rep("sensor2ego"), g["camera2imgs"][:1], rep("post_rots"), rep("post_trans"))
    assert (np.abs(P - ref).reshape(-1, 12).max(1) / np.abs(ref).reshape(-1, 12).max(1)).max() < 1.2e-7
