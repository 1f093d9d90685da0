"""Runtime backends of the Qwen3.8 family: shape rules, padding cost, one-time binding; CPU forward stays usable."""
import pytest
import torch

from archlab_b200.models.qwen38 import Qwen38Config, Qwen38LM
from archlab_b200.models import qwen38_runtime as rt


def test_shape_rules_name_the_bf16_exceptions():
    tiny = Qwen38Config.for_scale("tiny")
    rules = rt.shape_rules(tiny, "nvfp4")
    assert rules["covered"] == [] and "gdn.qkv" in rules["bf16_exceptions"]          # nothing at width 64 is 128-aligned
    assert rt.shape_rules(tiny, "kernels_bf16")["bf16_exceptions"] == {}
    aligned = Qwen38Config.for_scale("tiny", hidden_size=128, intermediate_size=256, attention_head_dim=32, linear_key_dim=64, linear_value_dim=32)
    rules = rt.shape_rules(aligned, "fp8_block")
    assert {"mlp.gate", "mlp.up", "mlp.down", "attention.out", "attention.q_gate", "gdn.z", "gdn.qkv"} <= set(rules["covered"])
    assert set(rules["bf16_exceptions"]) == {"attention.k", "attention.v"}                  # 2 KV heads x 32 = 64 columns
    with pytest.raises(ValueError, match="runtime_backend"):
        rt.shape_rules(tiny, "te_fp4")


def test_expert_padding_counts_whole_tiles():
    cost = rt.expert_padding([0, 1, 128, 129, 300])
    assert cost == {"rows": 558, "padded_rows": 128 + 128 + 256 + 384, "tiles": 7, "overhead": (896 - 558) / 558}
    assert rt.expert_padding([])["overhead"] == 0.0


@pytest.mark.parametrize("backend", ["native", "fp8_block", "nvfp4"])
def test_binding_is_reported_once_and_the_model_still_steps(backend):
    torch.manual_seed(0)
    c = Qwen38Config.for_scale("tiny", hidden_size=128, intermediate_size=256, attention_head_dim=32, linear_key_dim=64, linear_value_dim=32)
    model = Qwen38LM(c)
    model.init_weights()
    report = rt.apply_runtime_backend(model, backend)
    if backend == "native":
        assert report["converted"] == []
    else:
        assert report["converted"] and all("lm_head" not in n for n in report["converted"])
        assert any("lm_head" in n for n in report["bf16_exceptions"])
        assert any(n.endswith("mlp.gate") for n in report["converted"]) and any(n.endswith("q_gate") for n in report["converted"])
        assert all(n.endswith((".k", ".v", ".ba")) or "lm_head" in n or "mtp" in n or "indexer" in n for n in report["bf16_exceptions"]), report["bf16_exceptions"]
    ids = torch.randint(0, c.vocab_size, (2, 16))
    loss = model(ids, ids)
    loss = loss[0] if isinstance(loss, tuple) else loss
    loss.backward()
    assert torch.isfinite(loss)
    with pytest.raises(ValueError, match="already runs"):
        rt.apply_runtime_backend(model, "native")
