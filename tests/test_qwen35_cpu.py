"""Qwen3.5 dense backbone with simplicial layers, inserted branches, and the determinant switch."""
import pytest
import torch

from archlab_b200.models import qwen35 as Q


def test_4b_geometry_and_layer_types():
    c = Q.Qwen35Config()
    assert (c.n_layer, c.hidden_size, c.n_heads, c.n_kv_heads, c.head_dim, c.intermediate_size, c.vocab_size) == (
        36, 2560, 32, 8, 128, 9728, 151936)
    assert [i for i in range(c.n_layer) if c.is_simplicial(i)] == list(range(3, 36, 4))
    assert (c.simplicial_w2, c.simplicial_w1) == (512, 32)


def test_tiny_backbone_learns():
    torch.manual_seed(0)
    m = Q.Qwen35LM(Q.Qwen35Config.tiny())
    m.init_weights()
    assert m.layer_types() == ["full_attention", "simplicial_attention"] * 2
    ids = torch.randint(0, 256, (2, 25))
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        loss = m(ids[:, :-1], ids[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]


def test_stratified_sites():
    types = ["linear_attention"] * 3 + ["full_attention"]
    types = types * 4
    sites = Q.stratified_sites(types, 0.25)
    assert sites == [4, 9, 14, 15]                              # 3 of 12 linear layers, 1 of 4 full layers
    assert len(Q.stratified_sites(types, 1.0)) == 16
    with pytest.raises(ValueError):
        Q.stratified_sites(types, 0.0)


@pytest.mark.parametrize("mechanism", ["simplicial", "local"])
def test_inserted_branches_start_as_identity_and_train_alone(mechanism):
    torch.manual_seed(0)
    m = Q.Qwen35LM(Q.Qwen35Config.tiny(simplicial_every=0))
    m.init_weights()
    ids = torch.randint(0, 256, (2, 17))
    before = m(ids)
    cfg = Q.InsertionConfig(hidden_size=64, mechanism=mechanism, query_heads=4, kv_heads=2, head_dim=16, short_window=2,
                            long_window=6)
    handles = Q.install(m, cfg, [1, 3], backend="reference")
    torch.testing.assert_close(m(ids), before)                  # zero output projection
    counts = Q.freeze_backbone(m)
    assert counts["trainable"] == 2 * cfg.branch_parameters()
    loss = m(ids[:, :-1], ids[:, 1:])
    loss.backward()
    assert m.inserted_branches["1"].output.weight.grad.abs().sum() > 0
    assert m.embed.weight.grad is None
    with pytest.raises(ValueError):
        Q.install(m, cfg, [0])
    info = Q.describe(cfg, [1, 3], m.layer_types())
    assert info["branch_parameters"] == counts["trainable"]
    for h in handles:
        h.remove()
    torch.testing.assert_close(m(ids), before)


def test_simplicial_switch_inherits_teacher():
    torch.manual_seed(0)
    sw = Q.SimplicialSwitch(24, n_heads=2, n_kv_heads=1, head_dim=12)
    x = torch.randn(1, 6, 24)
    sw.inherit(torch.randn(24, 24), torch.randn(12, 24), torch.randn(12, 24), torch.randn(24, 24))
    y = sw(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    y.sum().backward()
    assert sw.k2.bias.grad is not None
