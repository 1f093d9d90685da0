"""Converted Limite served from paged caches: prefill + batched decode reproduce the full forward; pages are returned."""
import pytest
import torch

from archlab_b200.models.limite import AdapterConfig, ConversionConfig, LimiteConfig, LimiteLM, install_adapters, replace_limite_attention
from archlab_b200.serve.limite_converted import ConvertedLimiteServer, ServingSettings, validate_serving


def converted():
    torch.manual_seed(0)
    m = LimiteLM(LimiteConfig.tiny(sliding_window=5))
    m.init_weights(0.05)
    replace_limite_attention(m, ConversionConfig(short_window=3, backend="reference"))
    with torch.no_grad():
        for b in m.layers:
            b.attn.short_kv_delta.normal_(std=0.05)
    return m.eval()


def test_prefill_and_batched_decode_match_the_full_forward():
    m = converted()
    a, b = torch.randint(0, 128, (14,)), torch.randint(0, 128, (9,))
    server = ConvertedLimiteServer(m, num_pages=8, max_context=256)
    free = server.free_pages()
    with torch.no_grad():
        la = server.prefill("a", a[:10])
        lb = server.prefill("b", b[:6])
        assert torch.allclose(la, m(a[:10].view(1, -1))[0, -1], atol=1e-4) and torch.allclose(lb, m(b[:6].view(1, -1))[0, -1], atol=1e-4)
        for step in range(3):
            out = server.decode(["a", "b"], torch.stack([a[10 + step], b[6 + step]]))
            assert torch.allclose(out[0], m(a[:11 + step].view(1, -1))[0, -1], atol=1e-4), step
            assert torch.allclose(out[1], m(b[:7 + step].view(1, -1))[0, -1], atol=1e-4), step
        only_a = server.decode(["a"], a[13:14])
        assert torch.allclose(only_a[0], m(a.view(1, -1))[0, -1], atol=1e-4)
    assert server.requests["a"].length == 14 and server.free_pages() == free - 2
    server.release("a"), server.release("b")
    assert server.free_pages() == free and not server.requests


def test_admission_rules():
    m = converted()
    server = ConvertedLimiteServer(m, num_pages=2, max_context=130)
    server.prefill("a", torch.randint(0, 128, (5,)))
    with pytest.raises(ValueError, match="prefilled once"):
        server.prefill("a", torch.randint(0, 128, (5,)))
    with pytest.raises(ValueError, match="does not fit"):
        server.prefill("b", torch.randint(0, 128, (131,)))
    with pytest.raises(ValueError, match="one token per distinct"):
        server.decode(["a", "a"], torch.zeros(2, dtype=torch.long))
    with pytest.raises(RuntimeError, match="out of cache pages"):
        server.prefill("c", torch.randint(0, 128, (129,)))
    assert server.free_pages() == 1                                        # the failed prefill gave its pages back
    for settings, message in ((ServingSettings(tensor_parallel=2), "TP = PP = 1"), (ServingSettings(chunked_prefill=True), "chunked prefill"),
                              (ServingSettings(prefix_caching=True), "unquantised"), (ServingSettings(cache_dtype="fp8"), "unquantised"),
                              (ServingSettings(speculative=True), "speculative")):
        with pytest.raises(ValueError, match=message):
            validate_serving(m, settings)
    with pytest.raises(ValueError, match="qualified for short window"):
        validate_serving(m, ServingSettings(), short_window=16)
    plain = LimiteLM(LimiteConfig.tiny()).eval()
    with pytest.raises(ValueError, match="attention replacement in every layer"):
        validate_serving(plain, ServingSettings())
    with pytest.raises(ValueError, match="eval mode"):
        ConvertedLimiteServer(converted().train(), num_pages=2, max_context=128)
