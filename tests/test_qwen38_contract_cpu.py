"""Closed-form parameter contract and pipeline split of the Qwen3.8 family."""
import pytest
import torch

from archlab_b200.models import qwen38_contract as qc
from archlab_b200.models.qwen38 import Qwen38Config, Qwen38LM


@pytest.mark.parametrize("overrides", [
    {},                                                                              # dense, GDN + gated attention, MTP
    {"n_experts": 8, "experts_top_k": 2, "moe_intermediate_size": 32, "sparse_top_k": 8, "ngram_size": 3, "ngram_head_vocab": 53,
     "ngram_dim": 8},                                                                # Flash-Next mechanisms
    {"mtp_fusion": True, "shared_expert_gated": False, "n_experts": 4, "moe_intermediate_size": 16},
    {"mtp_layers": 0, "full_attention_interval": 2},
])
def test_contract_matches_the_built_model(overrides):
    cfg = Qwen38Config.for_scale("tiny", **overrides)
    with torch.device("meta"):
        model = Qwen38LM(cfg)
    want = qc.assert_parameter_contract(model)
    assert want["total"] == sum(p.numel() for p in model.parameters()) and len(want["per_layer"]) == cfg.num_hidden_layers


def test_published_scales_have_the_expected_size():
    full = qc.parameter_count_contract(Qwen38Config.for_scale("full"))
    assert 26e9 < full["total"] < 29e9                                              # the 27B text model
    quarter = qc.parameter_count_contract(Qwen38Config.for_scale("quarter"))
    assert quarter["total"] < full["total"] / 20


def test_pipeline_split_is_contiguous_and_balanced():
    cfg = Qwen38Config.for_scale("full")
    for stages in (1, 2, 4, 8):
        plan = qc.pipeline_split(cfg, stages)
        assert plan[0]["first_layer"] == 0 and plan[-1]["last_layer"] == cfg.num_hidden_layers
        assert all(a["last_layer"] == b["first_layer"] for a, b in zip(plan, plan[1:])) and all(p["last_layer"] > p["first_layer"] for p in plan)
        assert sum(p["parameters"] for p in plan) == qc.parameter_count_contract(cfg)["total"]
        if stages > 1:
            loads = [p["parameters"] for p in plan]
            assert max(loads) < 1.35 * (sum(loads) / stages)
            # the ends carry the embedding / head, so they get fewer layers than the middle stages
            assert plan[0]["last_layer"] - plan[0]["first_layer"] <= plan[1]["last_layer"] - plan[1]["first_layer"] or stages == 2
    with pytest.raises(ValueError):
        qc.pipeline_split(cfg, 0)
    tiny = Qwen38Config.for_scale("tiny")
    model = Qwen38LM(tiny)
    model.token_embedding = torch.nn.Embedding(tiny.vocab_size + 1, tiny.hidden_size)
    with pytest.raises(ValueError, match="promises"):
        qc.assert_parameter_contract(model)
