"""Width / depth scaling of the released V4.1 geometry; vectors from the reference's tests
(tests/test_deepseek_v41_scaling.py:47-76, tests/test_deepseek_v41_scratch.py:34-50)."""
import copy
from fractions import Fraction

import pytest

from archlab_b200.models import v41_scaling as vs


def released():
    return {"text_config": {
        "hidden_size": 5120, "num_hidden_layers": 40, "moe_intermediate_size": 2304, "head_dim": 512, "qk_rope_head_dim": 64,
        "q_lora_rank": 1280, "o_lora_rank": 1024, "index_head_dim": 128, "engram_head_dim": 256,
        "compress_ratios": [0, 0] + [2] * 18 + [1] * 20, "kv_source_layer_ids": [2, 8, 14, 20],
        "index_source_layer_ids": [2, 8, 14, 20, 24, 28, 32, 36], "engram_layer_ids": [1, 14], "candidate_source_layer_id": 20,
        "n_shared_experts": 1, "n_routed_experts": 384, "num_experts_per_tok": 6, "num_attention_heads": 64,
        "engram_num_embeddings": [384006168, 384016682], "engram_vocab_size": 1000, "engram_max_ngram_size": 3, "engram_n_heads": 2}}


@pytest.mark.parametrize("width,channels,adapter_dim", [
    (128, [128, 128, 16, 2, 32, 32, 4, 8], 16), (384, [384, 128, 64, 6, 96, 80, 16, 24], 16),
    (640, [640, 128, 64, 8, 160, 128, 16, 32], 16), (1280, [1280, 128, 128, 16, 320, 256, 32, 64], 32)])
def test_study_geometry(width, channels, adapter_dim):
    base = released()
    before = copy.deepcopy(base)
    text = vs.scaled_config(base, width=width, study=True)["text_config"]
    assert [text[k] for k in vs.CHANNEL_FIELDS] == channels and vs.adapter_head_dim(width) == adapter_dim
    assert text["num_hidden_layers"] == 20 and base == before
    for key in ("n_routed_experts", "n_shared_experts", "num_attention_heads", "engram_num_embeddings"):
        assert text[key] == base["text_config"][key]
    assert Fraction((text["num_experts_per_tok"] + 1) * text["moe_intermediate_size"], width) == 3
    assert text["qk_rope_head_dim"] % 2 == 0 and text["qk_rope_head_dim"] <= min(text["head_dim"], text["index_head_dim"])


def test_plain_eighth_scale_and_depth_resampling():
    base = released()
    out = vs.scaled_config(base)
    text = out["text_config"]
    assert all(text[k] * 8 == base["text_config"][k] for k in vs.CHANNEL_FIELDS)
    assert text["num_experts_per_tok"] == 6 and len(text["compress_ratios"]) == 20
    assert text["kv_source_layer_ids"] == [1, 4, 7, 10] and text["engram_layer_ids"] == [0, 7] and text["candidate_source_layer_id"] == 10
    assert vs.adapter_sites() == (2, 4, 7, 9, 12, 14, 17, 19) and "quantization_config" not in out
    deep = vs.scaled_config(base, depth=45)["text_config"]
    assert len(deep["compress_ratios"]) == 45 and deep["compress_ratios"][:3] == [0, 0, 0] and max(deep["index_source_layer_ids"]) < 45


@pytest.mark.parametrize("width", [0, True, 128.0, 256, 5120])
def test_undeclared_widths_are_refused(width):
    with pytest.raises(ValueError, match="scratch width"):
        vs.scaled_config(released(), width=width)


def test_other_refusals_and_engram_scaling():
    with pytest.raises(ValueError, match="depth"):
        vs.scaled_config(released(), depth=9)
    with pytest.raises(ValueError, match="requires scale_engram"):
        vs.scaled_config(released(), engram_anchor_width=128)
    wrong = released()
    wrong["text_config"]["hidden_size"] = 4096
    with pytest.raises(ValueError, match="released geometry"):
        vs.scaled_config(wrong)
    assert vs.routed_top_k(256, sweep=True) == 5
    scaled = vs.scaled_config(released(), width=640, scale_engram=True)["text_config"]
    assert scaled["engram_head_dim"] == 32 and scaled["engram_vocab_size"] == 125 and len(scaled["engram_num_embeddings"]) == 2
    fixed = vs.scaled_config(released(), width=1280, scale_engram=True, engram_anchor_width=640)["text_config"]
    assert fixed["engram_vocab_size"] == 125 and fixed["hidden_size"] == 1280


def test_a_scaled_geometry_builds_and_steps():
    import torch

    from archlab_b200.models.deepseek_v41 import V41LM

    text = vs.scaled_config(released(), width=128, depth=10, study=True)["text_config"]
    config = vs.to_model_config(text, vocab_size=128, sequence_len=32, n_routed_experts=8, n_heads=4, index_top_k=8, fp8_block=32)
    assert (config.hidden_size, config.n_layer, config.moe_inter, config.experts_top_k, config.head_dim, config.rope_dim) == (128, 10, 128, 2, 16, 2)
    model = V41LM(config)
    model.init_weights()
    ids = torch.randint(0, 128, (2, 16))
    loss = model(ids, ids)
    loss.backward()
    assert torch.isfinite(loss)
