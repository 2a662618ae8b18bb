"""Definitions in ``ops/reference.py`` against the library forms they restate."""
import torch


def test_causal_conv1d_silu_definition_matches_the_library_convolution():
    import torch.nn as nn
    from cppmega_b200.ops import functional as F_
    torch.manual_seed(0)
    conv = nn.Conv1d(24, 24, 4, groups=24, padding=3, bias=True)
    x = torch.randn(2, 37, 24)
    want = torch.nn.functional.silu(conv(x.transpose(1, 2))[..., :37]).transpose(1, 2)
    got = F_.causal_conv1d_silu(x, conv.weight, conv.bias)
    assert torch.allclose(got, want, atol=1e-6)
    # causal: the output at position s does not see later inputs
    x2 = x.clone()
    x2[:, 20:] += 1.0
    got2 = F_.causal_conv1d_silu(x2, conv.weight, conv.bias)
    assert torch.equal(got2[:, :20], got[:, :20])
