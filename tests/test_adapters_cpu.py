"""Stream adapters start as the identity, every mechanism trains and is causal; the triadic switch starts as its teacher."""
import pytest
import torch

from archlab_b200.models import adapters as A


def _cfg(m):
    return A.AdapterConfig(hidden_size=32, streams=4, mechanism=m, heads=2, kv_heads=1, head_dim=16, short_window=4, long_window=8,
                           low_rank=8, feature_rank=16, triadic_slices=2)


@pytest.mark.parametrize("m", A.MECHANISMS)
def test_adapter_identity_at_init_then_trains_causally(m):
    torch.manual_seed(0)
    ad = A.StreamAdapter(_cfg(m))
    packed = torch.randn(2, 12, 4 * 32)
    assert torch.allclose(ad(packed), packed)                       # zero-initialised output projection
    with torch.no_grad():
        ad.output.weight.normal_(0, 0.1)
    out = ad(packed)
    out.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in ad.parameters() if p.requires_grad)
    p2 = packed.clone()
    p2[:, 8] += 1.0
    with torch.no_grad():
        a, b = ad(packed), ad(p2)
    assert torch.allclose(a[:, :8], b[:, :8], atol=1e-5) and not torch.allclose(a[:, 8:], b[:, 8:])


def test_controls_are_parameter_matched():
    rep = A.parameter_report(A.AdapterConfig(hidden_size=64, heads=2, kv_heads=1, head_dim=32, low_rank=8, feature_rank=32))
    base = rep["simplicial"]
    assert abs(rep["normal"] - base) / base < 0.02 and abs(rep["mixer"] - base) / base < 0.05
    with pytest.raises(ValueError):
        A.AdapterConfig(hidden_size=8, mechanism="nope")


def test_triadic_switch_starts_as_the_teacher():
    torch.manual_seed(1)
    teacher = A.PlainDeltaMixer(24, 2, 8, 8)
    sw = A.TriadicSwitch(24, 2, 8, 8, slices=3)
    sw.inherit(teacher)
    x = torch.randn(2, 10, 24)
    assert torch.allclose(sw(x), teacher(x), atol=1e-5)
    sw(x).square().mean().backward()
    assert sw.k2.weight.grad is not None
