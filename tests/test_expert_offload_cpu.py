"""Host-offloaded experts: byte-bounded LRU, training-time arithmetic, encoded-row lookup."""
import pytest
import torch

from archlab_b200.models import moe
from archlab_b200.serve.expert_offload import DecodedExpertCache, OffloadedExperts, encoded_row_lookup


def decode(w, s):
    return w.float() * s


def test_cache_is_bounded_in_bytes_and_lru():
    enc = lambda v: {"a": (torch.full((4, 4), float(v)), torch.ones(1))}             # 64 bytes decoded
    cache = DecodedExpertCache(130, decode)
    for k in (1, 2):
        cache.get(k, enc(k))
    cache.get(1, enc(1))                                                                # 1 becomes most recent
    cache.get(3, enc(3))                                                                # evicts 2
    assert list(cache.entries) == [1, 3] and cache.stats() == {"hits": 1, "misses": 3, "evictions": 1, "resident_experts": 2, "resident_bytes": 128, "hit_rate": 0.25}
    big = {"a": (torch.zeros(8, 8), torch.ones(1))}                                     # 256 bytes: served, never kept
    assert cache.get("big", big)["a"].shape == (8, 8) and "big" not in cache.entries and cache.bytes <= 130


def test_offloaded_experts_match_the_training_layer():
    torch.manual_seed(0)
    experts = moe.GroupedExperts(4, 8, 6, swiglu_limit=7.0)
    experts.init_weights(0.3)
    x = torch.randn(10, 8)
    idx = torch.stack([torch.randperm(4)[:2] for _ in range(10)])
    prob = torch.rand(10, 2)
    tok = torch.arange(10).repeat_interleave(2)
    want = torch.zeros(10, 8).index_add_(0, tok, experts(x[tok], idx.flatten(), prob.flatten()[:, None]).float())
    gu, dn = experts.gate_up.detach(), experts.down.detach()
    encoded = [{"gate_up": ((gu[e] if gu[e].shape[-1] == 8 else gu[e].T).contiguous() / 2, torch.tensor(2.0)),
                "down": ((dn[e] if dn[e].shape[0] == 8 else dn[e].T).contiguous() / 2, torch.tensor(2.0))} for e in range(4)]
    layer = OffloadedExperts("L0", encoded, DecodedExpertCache(1 << 20, decode), swiglu_limit=7.0)
    got = layer(x, idx, prob)
    assert torch.allclose(got, want, atol=1e-5) and layer.cache.stats()["misses"] == len(torch.unique(idx))
    layer(x, idx, prob)
    assert layer.cache.stats()["hits"] == len(torch.unique(idx))


def test_encoded_rows_are_decoded_after_the_gather():
    torch.manual_seed(1)
    table = torch.randn(12, 8)
    scales = table.view(12, 2, 4).abs().amax(-1) / 448
    payload = (table.view(12, 2, 4) / scales[..., None]).flatten(1).to(torch.float8_e4m3fn)
    ids = torch.tensor([[0, 5], [11, 5]])
    got = encoded_row_lookup(payload, scales, ids, block=4, dim=8, out_dtype=torch.float32)
    want = (payload.float().view(12, 2, 4) * scales[..., None]).flatten(1)[ids]
    assert got.shape == (2, 2, 8) and torch.equal(got, want) and torch.allclose(got, table[ids], atol=0.15)
    with pytest.raises(ValueError, match="outside the original table"):
        encoded_row_lookup(payload, scales, torch.tensor([12]), block=4, dim=8)
