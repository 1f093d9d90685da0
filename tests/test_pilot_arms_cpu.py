"""Matched-control pilot arms: shared weights, seeded extras, arm semantics."""
import pytest
import torch

from archlab_b200.models import pilot_arms as pa
from archlab_b200.models.qwen35 import Qwen35Config


def _cfg():
    return Qwen35Config.tiny(n_layer=4, sequence_len=32)


def test_arms_share_common_weights_and_extras_are_counted():
    torch.manual_seed(7)
    before = torch.rand(1)
    torch.manual_seed(7)
    models = {arm: pa.build_arm(_cfg(), arm, seed=3, layers=(1, 3), short_window=2, long_window=8) for arm in pa.ARMS}
    digest = pa.assert_matched(models)
    assert len(digest) == 64
    count = lambda m: sum(p.numel() for p in m.parameters())
    assert count(models["A"]) == count(models["B"]) and count(models["C"]) - count(models["A"]) == models["C"].pilot["extra_parameters"] > 0
    assert models["B"].layer_types() == ["full_attention", "local_attention", "full_attention", "local_attention"]
    # the same seed gives the same extras, another seed other extras but the same closed-form count
    again = pa.build_arm(_cfg(), "C", seed=3, layers=(1, 3), short_window=2, long_window=8)
    assert pa.parameter_hashes(again) == pa.parameter_hashes(models["C"])
    other = pa.build_arm(_cfg(), "C", seed=4, layers=(1, 3), short_window=2, long_window=8)
    with pytest.raises(ValueError, match="do not share"):
        pa.assert_matched({"A": models["A"], "C": other})
    # installing the extras does not move the caller's RNG stream
    torch.manual_seed(7)
    m = pa.build_arm(_cfg(), "A", seed=3)
    torch.manual_seed(7)
    _ = torch.rand(1)
    assert torch.equal(before, _)


def test_arm_semantics():
    ids = torch.randint(0, 256, (2, 24), generator=torch.Generator().manual_seed(0))
    a = pa.build_arm(_cfg(), "A", seed=1, layers=(1,), short_window=2, long_window=4)
    b = pa.build_arm(_cfg(), "B", seed=1, layers=(1,), short_window=2, long_window=4)
    wide = pa.build_arm(_cfg(), "B", seed=1, layers=(1,), short_window=2, long_window=64)
    with torch.no_grad():
        ya, yb, yw = a(ids), b(ids), wide(ids)
    assert torch.allclose(ya, yw, atol=1e-5)                       # a window that covers the sequence is global attention
    assert not torch.allclose(ya, yb, atol=1e-4)
    assert torch.allclose(ya[:, :4], yb[:, :4], atol=1e-5)         # the first long_window positions see the same keys
    c = pa.build_arm(_cfg(), "C", seed=1, layers=(1,), short_window=2, long_window=4)
    loss = c(ids, labels=ids)
    loss.backward()
    grads = {n: p.grad for n, p in c.named_parameters() if ".attn.k2." in n or ".attn.v2." in n}
    assert len(grads) == 2 and all(g is not None and g.abs().sum() > 0 for g in grads.values())
    with pytest.raises(ValueError):
        pa.build_arm(_cfg(), "D")
    with pytest.raises(ValueError, match="windows"):
        pa.build_arm(_cfg(), "B", short_window=8, long_window=4)
    assert pa.pilot_layers(12) == (3, 7, 11)
