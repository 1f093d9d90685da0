"""Models built on the meta device get every parameter from ``init_weights``: nothing keeps allocator garbage."""
import pytest
import torch

from archlab_b200.models.factory import classes_for

SMALL = {
    "nanochat": dict(n_layer=2, n_embd=64, n_head=2, n_kv_head=2, vocab_size=256, sequence_len=32),
    "mhc": dict(n_layer=2, n_embd=64, n_head=2, n_kv_head=2, vocab_size=256, sequence_len=32),
    "kimi_kda": dict(n_layer=4, n_embd=64, n_head=2, vocab_size=256, sequence_len=32),
    "kimi_attnres": dict(n_layer=4, n_embd=64, n_head=2, vocab_size=256, sequence_len=32, attnres_block=2),
    "qwen35": None, "qwen38_tiny": None, "deepseek_v41": None,
}


@pytest.mark.parametrize("family", sorted(SMALL))
def test_init_weights_covers_every_parameter(family):
    cfg_cls, model_cls = classes_for(family)
    kw = SMALL[family]
    if kw is None:
        if not hasattr(cfg_cls, "tiny"):
            pytest.skip("no small configuration of this family")
        cfg = cfg_cls.tiny()
    else:
        cfg = cfg_cls(**kw)
    with torch.device("meta"):
        model = model_cls(cfg)
    if sum(p.numel() for p in model.parameters()) > 50_000_000:
        pytest.skip("small configuration is still large")
    model.to_empty(device="cpu")
    for p in model.parameters():
        p.data.fill_(float("nan"))
    model.init_weights()
    bad = [n for n, p in model.named_parameters() if not torch.isfinite(p).all()]
    assert not bad, bad[:10]
