"""Every frontier variant builds, trains one step, is causal, and its distinctive mechanism behaves."""
import pytest
import torch

from archlab_b200.models import frontier as fr


@pytest.mark.parametrize("variant", fr.VARIANTS)
def test_variant_trains_and_is_causal(variant):
    torch.manual_seed(0)
    cfg = fr.FrontierConfig.tiny(variant=variant, n_layer=4 if variant == "qwen_gdn" else 2, hc_anneal_steps=1)
    m = fr.FrontierLM(cfg)
    m.init_weights(0.05)
    ids = torch.randint(0, cfg.vocab_size, (2, 24))
    loss = m(ids[:, :-1], ids[:, 1:])
    loss.backward()
    assert torch.isfinite(loss) and all(p.grad is None or torch.isfinite(p.grad).all() for p in m.parameters())
    with torch.no_grad():
        a = m(ids[:, :-1])
        ids2 = ids.clone()
        ids2[:, 15] = (ids2[:, 15] + 1) % cfg.vocab_size
        b = m(ids2[:, :-1])
    assert torch.allclose(a[:, :15], b[:, :15], atol=1e-5) and not torch.allclose(a[:, 15:], b[:, 15:])


def test_short_conv_is_residual_and_causal():
    conv = fr.ShortConv(6, 4)
    x = torch.randn(1, 10, 6)
    y = conv(x)
    with torch.no_grad():
        conv.weight.zero_()
    assert torch.allclose(conv(x), x)
    x2 = x.clone()
    x2[:, 7] += 1
    assert torch.allclose(conv(x2)[:, :7], conv(x)[:, :7]) and y.shape == x.shape


def test_compressed_attention_sees_only_finished_blocks():
    cfg = fr.FrontierConfig.tiny(variant="deepseek_csa")
    att = fr.CompressedAttention(cfg, 0, heavy=False)
    assert att.m == 4 and fr.CompressedAttention(cfg, 0, heavy=True).m == 128
    comp = att._compress(torch.randn(1, 10, cfg.n_embd))
    assert comp.shape == (1, 3, cfg.head_dim) and torch.isfinite(comp).all()


def test_config_validation():
    with pytest.raises(ValueError):
        fr.FrontierConfig.tiny(variant="nope")
    with pytest.raises(ValueError):
        fr.FrontierConfig.tiny(variant="partial_rope_25", n_embd=48, n_head=4)       # head_dim 12 -> rotary width 3
