"""Host-side checks of the SamplingVT mirror that need no GPU: the 1x1 heads and their memory layout."""
import torch

from flashbev_b200.sampling_vt import SamplingVT

GRID = {"x": [-10, 10, 1.0], "y": [-10, 10, 1.0], "z": [-2, 2, 1.0], "depth": [1.0, 30.0, 1.0]}


def make(**kw):
    torch.manual_seed(3)
    return SamplingVT(GRID, (64, 176), in_channels=32, out_channels=16, **kw)


def test_heads_equal_the_convolutions_and_are_channels_last_in_memory():
    m = make()
    x = torch.randn(6, 32, 4, 11)
    for xin in (x, x.contiguous(memory_format=torch.channels_last)):
        f = m._pointwise_conv(m.context_network, xin)
        assert f.shape == (6, 16, 4, 11)
        assert torch.allclose(f, m.context_network(x), atol=2e-6)
        # what the operator is handed (sampling_vt.py:252-253) is already contiguous: no transpose kernel
        assert f.movedim(-3, -1).is_contiguous()
        d = m.forward_depth(xin)
        ref = m.depth_network(x) + torch.tensor([0.0, 0.1]).view(1, 2, 1, 1)
        assert torch.allclose(d, ref, atol=2e-6) and d.movedim(-3, -1).is_contiguous()


def test_heads_train():
    m = make()
    x = torch.randn(2, 32, 4, 11, requires_grad=True)
    (m._pointwise_conv(m.context_network, x).square().sum() + m.forward_depth(x).sum()).backward()
    ref = make()
    x2 = x.detach().clone().requires_grad_(True)
    (ref.context_network(x2).square().sum() + ref.depth_network(x2).sum()).backward()
    assert torch.allclose(x.grad, x2.grad, atol=1e-5)
    assert torch.allclose(m.context_network.weight.grad, ref.context_network.weight.grad, atol=1e-4)
    assert torch.allclose(m.depth_network[0].bias.grad, ref.depth_network[0].bias.grad, atol=1e-5)


def test_parameter_names_match_the_reference_module():
    # sampling_vt.py:172-180: context_network, depth_network.0, buffers depth_bins / roi_ranges / *_grid_size
    keys = set(make().state_dict())
    assert {"context_network.weight", "context_network.bias", "depth_network.0.weight", "depth_network.0.bias",
            "depth_bins", "roi_ranges", "output_grid_size", "sample_grid_size"} <= keys


# ---- against a recorded run of the reference's own module (tests/golden/module_dense_*.npz) ----
import numpy as np  # noqa: E402
import pytest  # noqa: E402

from tests.helpers import MODULE_GRID, harness_metrics, harness_pass, module_golden  # noqa: E402


@pytest.mark.parametrize("dist", ["laplace", "gaussian"])
def test_dense_branch_reproduces_the_reference_module(dist):
    """State dict of the reference module (dense branch) loaded into this module's dense branch on the CPU: same
    heads, same BEV features at the reference harness's own tolerances (tools/profile_differences.py:75-77,104)."""
    inputs, state, image, bev_ref, depths_ref = module_golden(dist)
    m = SamplingVT(MODULE_GRID, image, downsample=16, in_channels=32, out_channels=16, fuse_projection=False,
                   use_bev_pool=False, depth_distribution=dist, depth_weight_threshold=0.0).eval()
    missing, unexpected = m.load_state_dict(state, strict=False)
    assert not unexpected and all(k.split(".")[0] not in ("context_network", "depth_network") for k in missing)
    with torch.no_grad():
        bev, depths = m(inputs)
    assert bev.shape == bev_ref.shape and depths.shape == depths_ref.shape
    assert np.abs(depths.numpy() - depths_ref).max() < 1e-5
    met = harness_metrics(bev.numpy(), bev_ref)
    assert harness_pass(met), met


@pytest.mark.parametrize("dist", ["laplace", "gaussian"])
def test_pillar_pool_lists_and_oracle_reproduce_the_reference_module(dist):
    """The pillar-pool baseline's host side (projection of every voxel, sample lists sorted by BEV cell, intervals)
    fed to the numpy restatement of its kernel gives the reference module's BEV features: without a weight
    threshold the baseline and the dense branch compute the same mean.  This pins the restatement."""
    from oracle import oracle as O
    from flashbev_b200.sampling_vt import create_projection_matrix, pillar_pool_lists, project_voxels
    inputs, state, image, bev_ref, _ = module_golden(dist)
    m = SamplingVT(MODULE_GRID, image, downsample=16, in_channels=32, out_channels=16, fuse_projection=False,
                   use_bev_pool=True, depth_distribution=dist, depth_weight_threshold=0.0).eval()
    m.load_state_dict(state, strict=False)
    with torch.no_grad():
        x = inputs[0].flatten(0, 1)
        feats = m._pointwise_conv(m.context_network, x)
        depths = m.forward_depth(x)
        P = create_projection_matrix(*inputs[1:7])
        c3 = m.coords_3d
        u, v, d = project_voxels(P, (c3[:, 0, 0, 0], c3[0, :, 0, 1], c3[0, 0, :, 2]))
        fu, fv, fd, cams, ranks, starts, lengths = pillar_pool_lists(u, v, d, image, feats.shape[-2:])
    B, (X, Y, _) = inputs[0].shape[0], m._grid
    assert int(lengths.sum()) == fu.numel() and bool((ranks[1:] >= ranks[:-1]).all())
    out = O.pillar_pool(depths.movedim(1, -1).numpy(), feats.movedim(1, -1).numpy(), fu.numpy(), fv.numpy(), fd.numpy(),
                        cams.numpy(), ranks.numpy(), starts.numpy(), lengths.numpy(), B * X * Y, dist == "laplace")
    bev = out.reshape(B, X, Y, -1).transpose(0, 3, 2, 1)   # [B,X,Y,C] -> [B,C,Y,X]
    met = harness_metrics(bev, bev_ref)
    assert harness_pass(met), met
