"""Continuous-batching engine over paged caches reproduces greedy decoding by full re-computation."""
import torch

from archlab_b200.models import limite as L
from archlab_b200.serve.engine import SimplicialServingEngine


def _greedy(model, prompt, n):
    ids = list(prompt)
    out = []
    with torch.no_grad():
        for _ in range(n):
            t = int(model(torch.tensor([ids]))[0, -1].argmax())
            out.append(t)
            ids.append(t)
    return out


def test_engine_matches_full_recomputation_and_recycles_pages():
    torch.manual_seed(0)
    m = L.LimiteLM(L.LimiteConfig.tiny(sliding_window=40))
    m.init_weights(0.2)
    L.replace_limite_attention(m, L.ConversionConfig(short_window=4))
    with torch.no_grad():
        for b in m.layers:
            b.attn.short_kv_delta.normal_(0, 0.05)              # a genuinely trilinear model, not the initial identity
    m.eval()
    eng = SimplicialServingEngine(m, num_pages=4, max_batch=2, max_seq_len=256)
    prompts = [torch.randint(0, 128, (n,)).tolist() for n in (5, 130, 17)]
    ids = [eng.add_request(p, 6) for p in prompts]
    stats = eng.step()
    assert stats["admitted"] == 2 and stats["waiting"] == 1      # batch limit: the third request waits
    out = eng.run_until_done()
    for rid, p in zip(ids, prompts):
        assert out[rid] == _greedy(m, p, 6), rid
    assert len(eng.free) == 4 and not eng.running and not eng.waiting


def test_serving_admission_rules():
    import pytest
    import torch

    from archlab_b200.models import limite as L
    from archlab_b200.serve.engine import ServingSettings, SimplicialServingEngine, validate_serving

    torch.manual_seed(0)
    m = L.LimiteLM(L.LimiteConfig.tiny())
    plain = L.LimiteLM(L.LimiteConfig.tiny())
    L.replace_limite_attention(m, L.ConversionConfig(short_window=3, backend="reference"))
    validate_serving(m, ServingSettings())
    for settings, message in ((ServingSettings(tensor_parallel=2), "TP = PP = 1"), (ServingSettings(chunked_prefill=True), "chunked prefill"),
                              (ServingSettings(prefix_caching=True), "unquantised"), (ServingSettings(cache_dtype="fp8"), "unquantised"),
                              (ServingSettings(speculative=True), "speculative"), (ServingSettings(quantization="awq"), "quantisation")):
        with pytest.raises(ValueError, match=message):
            validate_serving(m, settings)
    with pytest.raises(ValueError, match="qualified for short window"):
        validate_serving(m, ServingSettings(), short_window=16)
    with pytest.raises(ValueError, match="attention replacement in every layer"):
        validate_serving(plain, ServingSettings())
    with pytest.raises(ValueError, match="chunked prefill"):
        SimplicialServingEngine(m, num_pages=2, settings=ServingSettings(chunked_prefill=True))
