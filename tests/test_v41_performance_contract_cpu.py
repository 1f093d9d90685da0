"""V4.1 performance contract: complete, typed, mutually consistent -- or refused."""
import json

import pytest

from archlab_b200.contracts.v41_performance import apply_to_config, read_performance_contract, trimmed_length

GOOD = {"format": "archlab-v41-performance-v1", "grouped_experts": True, "scale_engram": True, "engram_optimizer": "sinkhorn-algorithm-1", "table_lr_scale": 0.5,
        "batched_updates": True, "optimized_synchronization": True, "trim_alignment": 512, "head_loss_chunk": 1024, "router_bias_rate": 0.001,
        "retain_activations": False, "compile_hc_backward": True, "expert_dispatcher": "peer", "microbatch": 8}


def write(tmp_path, **edit):
    body = {k: v for k, v in {**GOOD, **edit}.items() if v is not ...}
    path = tmp_path / "perf.json"
    path.write_text(json.dumps(body))
    return path


def test_a_complete_contract_maps_onto_settings(tmp_path):
    assert read_performance_contract(None) is None and apply_to_config(None) == {}
    contract = read_performance_contract(write(tmp_path))
    settings = apply_to_config(contract)
    assert settings["model"]["use_peer_expert_parallel"] and settings["trainer"] == {"micro_batch": 8, "head_loss_chunk": 1024, "trim_alignment": 512,
                                                                                      "activation_checkpointing": True}
    assert settings["model"]["simplicial_deterministic"] is True
    v2 = read_performance_contract(write(tmp_path, format="archlab-v41-performance-v2", engram_anchor_width=128, simplicial_backend="kernel"))
    assert apply_to_config(v2)["model"]["engram_anchor_width"] == 128 and apply_to_config(v2)["model"]["simplicial_deterministic"] is False
    assert trimmed_length(4100, 512) == 4096
    with pytest.raises(ValueError):
        trimmed_length(100, 512)


@pytest.mark.parametrize("edit,message", [({"microbatch": 6}, "micro-batch"), ({"trim_alignment": 100}, "compression alignment"), ({"head_loss_chunk": 64}, "head chunk"),
                                          ({"router_bias_rate": 0.1}, "router rate"), ({"table_lr_scale": 0}, "learning-rate scale"),
                                          ({"grouped_experts": 1}, "must be boolean"), ({"scale_engram": False}, "scaled Engram"),
                                          ({"expert_dispatcher": "peer", "grouped_experts": False}, "requires grouped experts"),
                                          ({"expert_dispatcher": "nccl"}, "unsupported expert dispatcher"), ({"format": "v0"}, "unrecognised"),
                                          ({"extra_knob": 1}, "unrecognised"), ({"microbatch": ...}, "unrecognised"),
                                          ({"format": "archlab-v41-performance-v2"}, "unrecognised"),
                                          ({"format": "archlab-v41-performance-v2", "engram_anchor_width": 256}, "width-128"),
                                          ({"simplicial_backend": "triton"}, "simplicial training backend")])
def test_refusals(tmp_path, edit, message):
    with pytest.raises(ValueError, match=message):
        read_performance_contract(write(tmp_path, **edit))
