"""Incremental stream adapter: chunked prefill + single-token decode equals the full-sequence forward; state is bounded."""
import pytest
import torch

from archlab_b200.models.adapters import AdapterConfig, StreamAdapter
from archlab_b200.serve.adapter_cache import IncrementalStreamAdapter


@pytest.mark.parametrize("mechanism", ["simplicial", "normal"])
def test_chunks_and_tokens_match_the_full_forward(mechanism):
    torch.manual_seed(0)
    c = AdapterConfig(hidden_size=32, streams=2, mechanism=mechanism, heads=2, kv_heads=1, head_dim=16, short_window=3, long_window=6, low_rank=8)
    adapter = StreamAdapter(c, seed=1).eval()
    torch.nn.init.normal_(adapter.output.weight, std=0.2)            # the branch must contribute for the test to mean anything
    packed = torch.randn(2, 17, 64)
    with torch.no_grad():
        want = adapter(packed)
    assert (want - packed).abs().max() > 1e-3
    inc = IncrementalStreamAdapter(adapter)
    got, at = [], 0
    for length in (5, 1, 1, 7, 1, 2):
        got.append(inc(packed[:, at:at + length], start_position=at))
        at += length
    assert torch.allclose(torch.cat(got, 1), want, atol=1e-5, rtol=1e-5)
    lengths = inc.cache_lengths
    assert max(lengths.values()) == c.long_window - 1 and inc.position == 17
    if mechanism == "simplicial":
        assert lengths["k0"] == c.short_window - 1 and lengths["k1"] == c.long_window - 1


def test_contract_violations_leave_the_state_alone():
    c = AdapterConfig(hidden_size=32, streams=2, mechanism="simplicial", heads=2, kv_heads=1, head_dim=16, short_window=3, long_window=6, low_rank=8)
    adapter = StreamAdapter(c).eval()
    inc = IncrementalStreamAdapter(adapter)
    inc(torch.randn(1, 4, 64), start_position=0)
    before = {k: v.clone() for k, v in inc._cache.items()}
    for bad, kwargs, message in ((torch.randn(1, 2, 64), {"start_position": 0}, "non-contiguous"),
                                 (torch.randn(2, 2, 64), {"start_position": 4}, "changed within"),
                                 (torch.randn(1, 2, 60), {"start_position": 4}, "expected unpadded")):
        with pytest.raises(ValueError, match=message):
            inc(bad, **kwargs)
    assert inc.position == 4 and all(torch.equal(before[k], inc._cache[k]) for k in before)
    adapter.train()
    with pytest.raises(ValueError, match="eval mode"):
        inc(torch.randn(1, 1, 64), start_position=4)
    with pytest.raises(TypeError):
        IncrementalStreamAdapter(StreamAdapter(AdapterConfig(hidden_size=32, streams=2, mechanism="mixer", low_rank=8)))
    inc.reset()
    assert inc.position == 0 and inc.cache_lengths == {}
