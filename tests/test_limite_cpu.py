"""Limite family: adapters leave the function unchanged at install, conversion to simplicial attention is
exact at initialisation, the FLOP ledger's closed forms, chunked head, static-cache decoding."""
import pytest
import torch

from archlab_b200.models import limite as L


def _model(**kw):
    torch.manual_seed(0)
    m = L.LimiteLM(L.LimiteConfig.tiny(**kw))
    m.init_weights(0.08)
    return m


def test_adapters_are_identity_at_install_and_trainable_modes():
    m = _model()
    ids = torch.randint(0, 128, (2, 20))
    before = m(ids)
    L.install_adapters(m, L.AdapterConfig(heads=2, head_dim=8, window=5))
    assert torch.allclose(m(ids), before, atol=1e-6)
    total = sum(p.numel() for p in m.parameters())
    n_adapter = L.set_trainable_mode(m, "adapter")
    assert 0 < n_adapter < total and L.set_trainable_mode(m, "full") == total
    assert set(L.adapter_state(m)) | set(L.backbone_state(m)) == set(m.state_dict())
    with pytest.raises(ValueError):
        L.install_adapters(m, L.AdapterConfig())


def test_conversion_is_exact_at_initialisation_then_trains():
    m = _model()
    ids = torch.randint(0, 128, (1, 24))
    before = m(ids)
    L.replace_limite_attention(m, L.ConversionConfig(short_window=4))
    assert torch.allclose(m(ids), before, atol=2e-5)
    meta = L.conversion_metadata(m)
    assert meta["converted_layers"] == 4 and meta["short_window"] == 4
    m(ids[:, :-1], ids[:, 1:]).backward()
    assert m.layers[0].attn.short_kv_delta.grad.abs().sum() > 0
    with pytest.raises(ValueError):
        L.replace_limite_attention(m, L.ConversionConfig())


def test_flop_ledger_closed_forms():
    for n, a, b in [(10, 3, 7), (5, 8, 8), (9, 4, 4), (6, 2, 50)]:
        assert L.causal_pairs(n, a) == sum(min(i + 1, a) for i in range(n))
        assert L.causal_triples(n, a, b) == sum(min(i + 1, a) * min(i + 1, b) for i in range(n))
    c = L.LimiteConfig.tiny()
    full, adapter = L.baseline_flops(c, 32, "full"), L.baseline_flops(c, 32, "adapter")
    assert adapter.linear_per_token * 6 == full.linear_per_token * 4 and adapter.attention_per_token == full.attention_per_token
    conv = L.converted_flops(L.LimiteConfig.tiny(conversion={"short_window": 4}), 32)
    assert conv.linear_per_token > full.linear_per_token and conv.attention_per_token > full.attention_per_token
    assert full.mfu(1000, 1.0, 1, peak=full.per_token * 1000) == pytest.approx(1.0)
    with pytest.raises(ValueError):
        L.converted_flops(c, 32)


def test_chunked_head_matches_unchunked_with_gradients():
    torch.manual_seed(1)
    head = torch.nn.Linear(16, 50, bias=False)
    hidden = torch.randn(2, 11, 16, requires_grad=True)
    labels = torch.randint(0, 50, (2, 11))
    temp = torch.rand(2, 11) + 0.5
    out = L.chunked_logits_processor(head, hidden, L.logprob_entropy_processor, {"labels": labels, "temperature": temp}, chunk_size=4)
    ref = L.logprob_entropy_processor(head(hidden), labels, temp)
    assert all(torch.allclose(out[k], ref[k], atol=1e-6) for k in ref)
    g1 = torch.autograd.grad(out["log_probs"].sum(), [hidden, head.weight])
    g2 = torch.autograd.grad(ref["log_probs"].sum(), [hidden, head.weight])
    assert all(torch.allclose(a, b, atol=1e-5) for a, b in zip(g1, g2))
    with pytest.raises(ValueError):
        L.chunked_logits_processor(head, hidden, L.logprob_entropy_processor, {}, chunk_size=4)


def test_static_cache_decoding_matches_full_forward():
    m = _model().eval()
    ids = torch.randint(0, 128, (2, 30))
    with torch.no_grad():
        full = m(ids)
        logits, ks, vs = L.prefill(m, ids[:, :12])
        assert torch.allclose(logits, full[:, 11], atol=1e-4)
        dec = L.GraphDecoderPool(m).get(2, 64)
        dec.reset(ks, vs, ids[:, 12:13])
        for t in range(12, 30):                                # crosses the sliding window (span 8) several times
            out = dec(ids[:, t:t + 1])
            assert torch.allclose(out, full[:, t], atol=1e-4), t


def test_conversion_backend_tri_state_and_fixed_scale_query_rule():
    import math

    import pytest

    torch.manual_seed(0)
    with pytest.raises(ValueError):
        L.ConversionConfig(backend="triton")
    ids = torch.randint(0, 128, (1, 10))
    outs = {}
    for backend in ("auto", "reference"):
        torch.manual_seed(1)
        m = L.LimiteLM(L.LimiteConfig.tiny())
        m.init_weights()
        L.replace_limite_attention(m, L.ConversionConfig(short_window=4, backend=backend))
        outs[backend] = m(ids)
    torch.testing.assert_close(outs["auto"], outs["reference"], rtol=1e-4, atol=1e-4)
    torch.manual_seed(1)
    m = L.LimiteLM(L.LimiteConfig.tiny())
    m.init_weights()
    L.replace_limite_attention(m, L.ConversionConfig(short_window=4, backend="kernel"))
    with pytest.raises(RuntimeError, match="kernel"):
        m(ids)                                           # CPU, fp32: the kernel backend must refuse, not fall back
    # a backend with a hard-coded D ** -0.5 realises `scaling` through a pre-scaled fp32 query
    from archlab_b200.ops.simplicial import simplicial_attention_reference as ref

    q, k = torch.randn(1, 6, 2, 16).bfloat16(), torch.randn(1, 6, 2, 16)
    scaling, fixed = 0.31, 1 / math.sqrt(16)
    pre = L.query_for_fixed_scale(q, scaling, fixed)
    assert pre.dtype == torch.float32
    a = ref(pre, k, k, k, k, 2, 4, scale=fixed)
    b = ref(q.float(), k, k, k, k, 2, 4, scale=scaling)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
