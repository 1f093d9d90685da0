"""SoTA component pool: each mechanism, the combinations, fake quantisation, CoLU, the quantisation monitor."""
import pytest
import torch

from archlab_b200.models import sota as S


@pytest.mark.parametrize("mech", [(), ("dyt",), ("xielu",), ("canon",), ("bov",), ("diff_attn",), ("gated_relu",), ("colu",), ("qat",),
                                  ("canon", "bov", "gated_relu")])
@pytest.mark.parametrize("fog", [None, "flash"])
def test_pool_trains_and_is_causal(mech, fog):
    if fog and "diff_attn" in mech:
        pytest.skip("FOG regularisation applies to the standard attention path")
    torch.manual_seed(0)
    cfg = S.SotaConfig.tiny(mechanisms=mech, fog_variant=fog)
    m = S.SotaLM(cfg)
    m.init_weights(0.05)
    ids = torch.randint(0, cfg.vocab_size, (2, 20))
    loss = m(ids[:, :-1], ids[:, 1:])
    loss.backward()
    assert torch.isfinite(loss)
    with torch.no_grad():
        a = m(ids[:, :-1])
        ids2 = ids.clone()
        ids2[:, 12] = (ids2[:, 12] + 3) % cfg.vocab_size
        b = m(ids2[:, :-1])
    assert torch.allclose(a[:, :12], b[:, :12], atol=1e-5) and not torch.allclose(a[:, 12:], b[:, 12:])


def test_bov_table_reproduces_projection_at_init():
    cfg = S.SotaConfig.tiny(mechanisms=("bov",))
    m = S.SotaLM(cfg)
    assert m.architecture_state()["bov_layers"] == [3]
    att, proj = m.layers[3].attn, torch.nn.Linear(64, 64, bias=False)
    att.init_bov(m.embed, proj)
    ids = torch.randint(0, 128, (1, 5))
    from archlab_b200.models.blocks import rms_norm
    assert torch.allclose(att.value_table(ids), proj(rms_norm(m.embed(ids))), atol=1e-6)


def test_fake_quantisation_and_ste():
    x = torch.randn(4, 32, requires_grad=True)
    y = S.fake_quant_int8_per_token(x)
    assert (y - x).abs().max() <= (x.amax(-1) - x.amin(-1)).max() / 255 + 1e-6
    y.sum().backward()
    assert torch.allclose(x.grad, torch.ones_like(x))
    w = torch.randn(6, 40)
    q = S.fake_quant_int4_per_group(w, 16)
    levels = (q.view(6, -1)[:, :16] / (w[:, :16].abs().amax(-1, keepdim=True) / 7)).round()
    assert q.shape == w.shape and levels.abs().max() <= 8 and levels.unique().numel() <= 16
    with pytest.raises(ValueError):
        S.fake_quant_int4_per_group(torch.randn(3), 4)


def test_colu_xielu_dyt_and_monitor():
    x = torch.randn(2, 3, 16)
    y = S.soft_colu(x, 4)
    assert y.shape == x.shape and torch.allclose(y[..., :4], torch.nn.functional.silu(x[..., :4]))
    act = S.XIELU()
    z = torch.tensor([-2.0, 0.5])
    assert torch.allclose(act(z)[1], 0.8 * z[1] ** 2 + 0.5 * z[1], atol=1e-6) and act(z)[0] < 0
    assert torch.allclose(S.DynamicTanh(4)(torch.zeros(4)), torch.zeros(4))
    assert S.matched_gated_width(768) == 2048 and S.matched_gated_width(64, 4) % 4 == 0
    m = S.SotaLM(S.SotaConfig.tiny(fog_variant="opt"))
    m.init_weights()
    m.monitor.set_enabled(True)
    m(torch.randint(0, 128, (1, 8)))
    rec = m.monitor.consume()
    assert "layer0/q/kurtosis" in rec and rec["layer0/q/nonfinite_frac"] == 0 and not m.monitor.consume()
    assert S.combo_config("canon_xielu", n_layer=2, n_embd=64, n_head=4, vocab_size=64).mechanisms == ("canon", "xielu")
    with pytest.raises(ValueError):
        S.SotaConfig.tiny(mechanisms=("colu", "xielu"))
