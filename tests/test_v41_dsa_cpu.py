"""DSA ops and the V4.1-style MoE LM on CPU."""
import torch

from archlab_b200.models.deepseek_v41 import V41Config, V41LM
from archlab_b200.ops import dsa


def test_sparse_attention_with_all_keys_equals_dense():
    torch.manual_seed(0)
    B, S, H, D = 2, 12, 3, 8
    q, kv, sink = torch.randn(B, S, H, D), torch.randn(B, S, D), torch.randn(H)
    w = torch.rand(B, S, 2)
    scores = dsa.indexer_scores(torch.randn(B, S, 2, 4), torch.randn(B, S, 4), w)
    idx, vals = dsa.select_topk(scores, S)
    assert ((idx >= 0).sum(-1) == torch.arange(1, S + 1)).all()         # causal: query t sees t+1 keys
    sparse = dsa.sparse_attention(q, kv, sink, idx, D ** -0.5, query_chunk=5)
    dense = dsa.dense_sink_attention(q, kv, sink, D ** -0.5)
    torch.testing.assert_close(sparse, dense, atol=1e-5, rtol=1e-5)
    rounded = dsa.sparse_attention(q, kv, sink, idx, D ** -0.5, native_rounding=True)
    assert (rounded - dense).abs().max() < 3e-2


def test_sink_takes_mass_and_duplicates_count():
    q, kv = torch.zeros(1, 1, 1, 4), torch.ones(1, 2, 4)
    idx = torch.tensor([[[0, 0, -1]]])
    out = dsa.sparse_attention(q, kv, torch.zeros(1), idx, 1.0)
    torch.testing.assert_close(out, torch.full((1, 1, 1, 4), 2.0 / 3.0))    # two unit slots + unit sink


def test_indexer_kl_zero_at_match_and_grad():
    s = torch.randn(2, 5, 5)
    valid = torch.ones(5, 5, dtype=torch.bool).tril().expand(2, 5, 5)
    target = s.masked_fill(~valid, float("-inf")).softmax(-1)
    assert dsa.indexer_kl(target, s, valid).abs() < 1e-6
    s2 = (s + torch.randn_like(s)).requires_grad_(True)
    kl = dsa.indexer_kl(target, s2, valid)
    assert kl > 0
    kl.backward()
    assert torch.isfinite(s2.grad).all()


def _train(model, steps=10):
    torch.manual_seed(0)
    ids = torch.randint(0, model.config.vocab_size, (2, 25))
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    out = []
    for _ in range(steps):
        loss = model(ids[:, :-1], ids[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        out.append(float(model.last_loss_metrics["cross entropy"]))
    return out


def test_v41_tiny_learns_sparse_and_fp8():
    for kw in ({}, {"fp8": True}):
        m = V41LM(V41Config.tiny(**kw))
        m.init_weights()
        losses = _train(m)
        assert losses[-1] < losses[0], (kw, losses)
        assert m.layers[0].attn.indexer.q_proj.weight.grad is not None       # learns from the KL only
        assert float(m.last_loss_metrics["indexer kl"]) >= 0


def test_hyper_connection_starts_near_identity_mixing():
    m = V41LM(V41Config.tiny())
    m.init_weights()
    pre, post, comb = m.layers[0].hc_attn.coefficients(torch.randn(1, 3, 4, 64))
    assert comb.shape == (1, 3, 4, 4)
    assert (comb.diagonal(dim1=-2, dim2=-1) > 0.8).all()
