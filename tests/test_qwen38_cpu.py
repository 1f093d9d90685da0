"""Qwen3.8 hybrid LM: dense, MoE/sparse/PLE variants train on CPU; contracts hold."""
import torch

from archlab_b200.models.qwen38 import GatedDeltaNet, Qwen38Config, Qwen38LM
from archlab_b200.ops import delta_rule


def _step(model, steps=8, lr=3e-3):
    torch.manual_seed(0)
    ids = torch.randint(1, model.config.vocab_size, (2, 33))
    x, y = ids[:, :-1], ids[:, 1:]
    opt = torch.optim.AdamW(model.parameters(), lr=lr)
    losses = []
    for _ in range(steps):
        loss = model(x, y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses


def test_dense_quarter_geometry_contract():
    c = Qwen38Config.for_scale("quarter")
    assert (c.num_hidden_layers, c.hidden_size, c.attention_head_dim) == (16, 1280, 64)
    f = Qwen38Config.for_scale("full")
    assert (f.num_hidden_layers, f.hidden_size, f.intermediate_size, f.attention_heads, f.attention_head_dim) == (
        64, 5120, 17408, 24, 256) and f.mtp_fusion


def test_tiny_dense_learns_and_tags_every_parameter():
    m = Qwen38LM(Qwen38Config.for_scale("tiny"))
    m.init_weights()
    kinds = [b.attention_kind for b in m.layers]
    assert kinds == ["gdn", "gdn", "gdn", "full_attention"]
    contract = m.optimizer_contract()
    assert set(contract["optimizers"]) == {"adamw", "muon"}
    total = sum(b["parameters"] for b in contract["optimizers"].values())
    assert total == m.num_scaling_params()["total"]
    losses = _step(m)
    assert losses[-1] < losses[0]
    assert set(m.last_loss_metrics) == {"cross entropy", "mtp loss"}
    logits = m(torch.randint(1, 512, (1, 9)))
    assert logits.shape == (1, 9, 512)


def test_mtp_fusion_and_loss_reductions():
    m = Qwen38LM(Qwen38Config.for_scale("tiny", mtp_fusion=True))
    m.init_weights()
    ids = torch.randint(1, 512, (2, 12))
    y = ids.clone()
    y[0, :3] = -1
    none = m(ids, y, loss_reduction="none")
    assert none.shape == ids.shape and (none[0, :3] == 0).sum() >= 0
    s, mean = m(ids, y, loss_reduction="sum"), m(ids, y)
    torch.testing.assert_close(mean, s / y.ne(-1).sum())


def test_moe_sparse_ple_variant_learns():
    c = Qwen38Config.for_scale("tiny", n_experts=4, experts_top_k=2, moe_intermediate_size=32, sparse_top_k=8,
                               indexer_heads=2, indexer_dim=8, ngram_size=3, ngram_head_vocab=101, ngram_dim=8)
    m = Qwen38LM(c)
    m.init_weights()
    losses = _step(m, steps=8)
    assert losses[-1] < losses[0]
    assert len(m.routers()) == 4 and m.routers()[0].last_metrics["load"].sum() == 2 * 32 * 2


def test_gdn_layer_matches_recurrent_oracle():
    c = Qwen38Config.for_scale("tiny")
    layer = GatedDeltaNet(c)
    torch.manual_seed(1)
    for p in layer.parameters():
        if p.ndim >= 2:
            torch.nn.init.normal_(p, std=0.2)
    x = torch.randn(2, 70, c.hidden_size)
    got = layer(x)
    orig = delta_rule.chunk_gated_delta_rule
    try:
        delta_rule.chunk_gated_delta_rule = lambda q, k, v, d, b, **kw: delta_rule.gated_delta_reference(q, k, v, d, b)
        want = layer(x)
    finally:
        delta_rule.chunk_gated_delta_rule = orig
    torch.testing.assert_close(got, want, atol=2e-4, rtol=1e-3)
