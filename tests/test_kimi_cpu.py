"""Kimi KDA / AttnRes model on CPU."""
import pytest
import torch

from archlab_b200.models import kimi
from archlab_b200.ops import delta_rule


def test_layer_map_pattern_and_final_global():
    m = kimi.kda_layer_map(8)
    assert m == {"kda": [1, 2, 3, 5, 6, 7], "global": [4, 8]}
    assert kimi.kda_layer_map(6)["global"] == [4, 6]          # last layer forced global
    with pytest.raises(ValueError):
        kimi.is_kda_layer(1, 4, "KXKG")


@pytest.mark.parametrize("variant", kimi.KDA_VARIANTS)
def test_kda_layer_matches_recurrence(variant):
    torch.manual_seed(0)
    c = kimi.KimiConfig(vocab_size=64, n_layer=4, n_head=2, n_embd=32, kda_variant=variant)
    layer = kimi.KimiDeltaAttention(c)
    for p in layer.parameters():
        if p.ndim >= 2:
            torch.nn.init.normal_(p, std=0.3)
    x = torch.randn(2, 70, 32)
    got = layer(x)
    orig = delta_rule.chunk_kda
    try:
        delta_rule.chunk_kda = lambda q, k, v, g, b, chunk=64: delta_rule.kda_recurrent_reference(q, k, v, g, b)
        want = layer(x)
    finally:
        delta_rule.chunk_kda = orig
    torch.testing.assert_close(got, want, atol=3e-4, rtol=1e-3)
    g = layer.gate(torch.randn(1, 3, 32))
    assert (g <= 0).all() and (variant != "kimi_k3" or (g >= -5).all())


def test_attnres_uniform_at_init_and_multihead():
    r = kimi.AttnResRead(8, heads=2)
    a, b = torch.randn(2, 3, 8), torch.randn(2, 3, 8)
    torch.testing.assert_close(r(a, b), (a + b) / 2)              # zero query: uniform softmax
    with torch.no_grad():
        r.query.normal_()
    out = r(a, b)
    assert out.shape == a.shape and not torch.allclose(out, (a + b) / 2)
    with pytest.raises(ValueError):
        r(a, torch.randn(2, 3, 4))


def test_kimi_lm_learns():
    torch.manual_seed(0)
    c = kimi.KimiConfig(vocab_size=64, sequence_len=32, n_layer=4, n_head=2, n_embd=32, attnres_block=2)
    m = kimi.KimiLM(c)
    m.init_weights()
    ids = torch.randint(0, 64, (2, 33))
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        loss = m(ids[:, :-1], ids[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]
