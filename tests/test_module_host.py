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
