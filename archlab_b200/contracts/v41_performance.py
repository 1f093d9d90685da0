"""The explicit opt-in contract of a V4.1 performance experiment: every speed-relevant switch is named in one JSON
document, or the run uses the plain defaults.  Nothing is inferred from the environment.

Keys (all required; unknown keys are refused):

    format                      "archlab-v41-performance-v1" | "-v2" (v2 adds ``engram_anchor_width``, which must be 128)
    grouped_experts             bool   grouped expert GEMMs instead of per-expert linears
    expert_dispatcher           "torch" | "peer"   ("peer": dispatch / combine kernels over peer memory; needs grouped experts)
    scale_engram                bool   must be true: the Sinkhorn table optimiser is defined for scaled tables
    engram_optimizer            "sinkhorn-algorithm-1"
    table_lr_scale              (0, 1]
    batched_updates             bool   packed statistics collective of the factored optimiser
    optimized_synchronization   bool
    trim_alignment              128 | 256 | 512 | 1024 | 2048   sequences are trimmed to this multiple (keeps compression blocks whole)
    head_loss_chunk             128 .. 2048   tokens per chunk of the full-vocabulary loss
    router_bias_rate            (0, 0.01]
    retain_activations          bool   keep instead of recompute
    compile_hc_backward         bool   fused hyper-connection coefficient backward
    microbatch                  4 | 8 | 16 | 32
    simplicial_backend          optional: "deterministic" (default) | "kernel"

``apply_to_config`` maps the contract onto ``V41Config`` / trainer arguments of this framework and returns what it set.
(Reference: src/archlab/automodel/deepseek_v41_performance.py:7-75.)
"""
from __future__ import annotations

import json
from pathlib import Path

FORMATS = ("archlab-v41-performance-v1", "archlab-v41-performance-v2")
BOOLEANS = ("grouped_experts", "scale_engram", "batched_updates", "optimized_synchronization", "retain_activations", "compile_hc_backward")
REQUIRED = frozenset({"format", *BOOLEANS, "engram_optimizer", "table_lr_scale", "trim_alignment", "head_loss_chunk", "router_bias_rate",
                      "expert_dispatcher", "microbatch"})
OPTIONAL = frozenset({"simplicial_backend"})


def read_performance_contract(path) -> dict | None:
    if path is None:
        return None
    value = json.loads(Path(path).read_text())
    version = value.get("format")
    required = REQUIRED | ({"engram_anchor_width"} if version == FORMATS[1] else set())
    if version not in FORMATS or set(value) - OPTIONAL != required:
        raise ValueError("unrecognised V4.1 performance contract")
    if version == FORMATS[1] and (type(value["engram_anchor_width"]) is not int or value["engram_anchor_width"] != 128):
        raise ValueError("the fixed Engram cohort requires the width-128 lookup budget")
    for key in BOOLEANS:
        if type(value[key]) is not bool:
            raise ValueError(f"{key} must be boolean")
    if value["engram_optimizer"] != "sinkhorn-algorithm-1" or not value["scale_engram"]:
        raise ValueError("this Sinkhorn contract requires scaled Engram tables")
    if type(value["trim_alignment"]) is not int or value["trim_alignment"] not in (128, 256, 512, 1024, 2048):
        raise ValueError("trimming must preserve compression alignment")
    if type(value["head_loss_chunk"]) is not int or not 128 <= value["head_loss_chunk"] <= 2048:
        raise ValueError("invalid full-vocabulary head chunk")
    if not 0 < value["table_lr_scale"] <= 1 or not 0 < value["router_bias_rate"] <= 0.01:
        raise ValueError("invalid table learning-rate scale or router rate")
    if value["expert_dispatcher"] not in ("torch", "peer"):
        raise ValueError("unsupported expert dispatcher")
    if value["expert_dispatcher"] == "peer" and not value["grouped_experts"]:
        raise ValueError("the peer-memory dispatcher requires grouped experts")
    if type(value["microbatch"]) is not int or value["microbatch"] not in (4, 8, 16, 32):
        raise ValueError("invalid controlled micro-batch")
    if value.get("simplicial_backend", "deterministic") not in ("deterministic", "kernel"):
        raise ValueError("unsupported simplicial training backend")
    return value


def trimmed_length(length: int, alignment: int) -> int:
    """Longest multiple of ``alignment`` not above ``length`` (at least one block)."""
    if length < alignment:
        raise ValueError("the sequence is shorter than one aligned block")
    return length // alignment * alignment


def apply_to_config(contract: dict | None) -> dict:
    """Trainer / model settings implied by the contract (empty without one)."""
    if contract is None:
        return {}
    return {"model": {"use_peer_expert_parallel": contract["expert_dispatcher"] == "peer", "grouped_experts": contract["grouped_experts"],
                      "router_bias_rate": contract["router_bias_rate"], "fused_hc_backward": contract["compile_hc_backward"],
                      "engram_anchor_width": contract.get("engram_anchor_width"),
                      "simplicial_deterministic": contract.get("simplicial_backend", "deterministic") == "deterministic"},
            "trainer": {"micro_batch": contract["microbatch"], "head_loss_chunk": contract["head_loss_chunk"], "trim_alignment": contract["trim_alignment"],
                        "activation_checkpointing": not contract["retain_activations"]},
            "optimizer": {"tables": contract["engram_optimizer"], "table_lr_scale": contract["table_lr_scale"], "batched_updates": contract["batched_updates"],
                          "overlapped_synchronization": contract["optimized_synchronization"]}}
