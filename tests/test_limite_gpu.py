"""Limite decode step captured in a CUDA graph reproduces the full forward; conversion runs the simplicial kernel."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_graph_decoder_replays_match_full_forward():
    from archlab_b200.models import limite as L

    torch.manual_seed(0)
    cfg = L.LimiteConfig.tiny(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128, intermediate_size=512,
                              sliding_window=15)
    m = L.LimiteLM(cfg)
    m.init_weights(0.05)
    m = m.cuda().bfloat16().eval()
    ids = torch.randint(0, 128, (2, 160), device="cuda")
    with torch.no_grad():
        full = m(ids)
        _, ks, vs = L.prefill(m, ids[:, :128])
        dec = L.GraphDecoder(m, 2, 256)
        dec.reset(ks, vs, ids[:, 128:129])
        assert dec.graph is not None
        for t in range(128, 160):
            out = dec(ids[:, t:t + 1])
            assert (out - full[:, t]).abs().max() < 0.15 * full[:, t].abs().max().clamp_min(1.0), t


def test_converted_model_trains_on_the_simplicial_kernel():
    from archlab_b200.models import limite as L
    from archlab_b200.ops import native

    torch.manual_seed(0)
    cfg = L.LimiteConfig.tiny(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128, intermediate_size=512,
                              sliding_window=127, global_layers=())
    m = L.LimiteLM(cfg)
    m.init_weights(0.05)
    m = m.cuda().bfloat16()
    ids = torch.randint(0, 128, (1, 257), device="cuda")
    with torch.no_grad():
        before = m(ids[:, :-1])
    L.replace_limite_attention(m, L.ConversionConfig(short_window=8))
    with torch.no_grad():
        after = m(ids[:, :-1])
    assert (after - before).abs().max() < 0.1 * before.abs().max()
    m(ids[:, :-1], ids[:, 1:]).backward()
    native.check_status()
    assert torch.isfinite(m.layers[0].attn.short_kv_delta.grad.float()).all()
