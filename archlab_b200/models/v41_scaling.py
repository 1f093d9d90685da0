"""Width / depth scaling of the released V4.1 geometry (hidden 5120, 40 layers) to randomly initialised study models.

Channels scale by ``width / 5120`` and round UP to what the kernels want (a table below: a multiple, and for the sparse
head dimensions a power of two); categorical counts (experts, heads, hash tables) stay.  Layer-indexed lists are
resampled to the new depth: per-layer lists pick the source layer ``i * 40 // depth``, "source layer" ids (which name
the first layer of a region) map by ceiling, engram sites by floor.  The scaling study fixes the expert width at 128
and picks the routed top-k so that active expert width (routed + the one shared expert) is exactly three times the
model width.  (Rule and golden vectors: src/archlab/architectures/deepseek_v41_scratch.py:45-118 and the reference's
tests/test_deepseek_v41_scaling.py:47-76, tests/test_deepseek_v41_scratch.py:34-50.)
"""
from __future__ import annotations

import copy
from fractions import Fraction

from .engram_geometry import scaled_engram_geometry

RELEASED_WIDTH, RELEASED_DEPTH = 5120, 40
STUDY_WIDTHS = (128, 384, 640, 1280)
SWEEP_WIDTHS = (128, 256, 384)
STUDY_EXPERT_WIDTH, STUDY_SHARED_EXPERTS, STUDY_ACTIVE_RATIO = 128, 1, 3
ADAPTER_SITES_RELEASED = (4, 9, 14, 19, 24, 29, 34, 39)

# channel -> (round up to a multiple of, then up to a power of two?)
CHANNEL_RULES = {
    "hidden_size": (1, False),
    "moe_intermediate_size": (16, False),
    "head_dim": (16, True),
    "qk_rope_head_dim": (2, False),
    "q_lora_rank": (16, False),
    "o_lora_rank": (16, False),
    "index_head_dim": (4, True),
    "engram_head_dim": (8, False),
}
CHANNEL_FIELDS = tuple(CHANNEL_RULES)


def _check_width(width, sweep: bool) -> None:
    if type(width) is not int or width not in (SWEEP_WIDTHS if sweep else STUDY_WIDTHS):
        raise ValueError(f"scratch width must be one of {SWEEP_WIDTHS if sweep else STUDY_WIDTHS}")


def scale_channel(value: int, width: int, multiple: int = 1, power_of_two: bool = False) -> int:
    exact = Fraction(value * width, RELEASED_WIDTH)
    units = -(-exact.numerator // (exact.denominator * multiple))            # ceil(exact / multiple)
    rounded = max(multiple, units * multiple)
    return 1 << (rounded - 1).bit_length() if power_of_two else rounded


def adapter_head_dim(width: int, *, sweep: bool = False) -> int:
    _check_width(width, sweep)
    return scale_channel(128, width, 16, True)


def routed_top_k(width: int, *, sweep: bool = False) -> int:
    _check_width(width, sweep)
    active = Fraction(STUDY_ACTIVE_RATIO * width, STUDY_EXPERT_WIDTH)
    if active.denominator != 1:
        raise ValueError("scratch width must make the active expert width a whole number of experts")
    return int(active) - STUDY_SHARED_EXPERTS


def adapter_sites(depth: int = 20) -> tuple[int, ...]:
    return tuple(site * depth // RELEASED_DEPTH for site in ADAPTER_SITES_RELEASED)


def scaled_config(released: dict, *, width: int = 640, depth: int = 20, study: bool = False, sweep: bool = False,
                  scale_engram: bool = False, engram_anchor_width: int | None = None) -> dict:
    """A complete model configuration (``text_config`` + an empty vision tower) for a study model; ``released`` is not
    modified."""
    _check_width(width, sweep)
    if type(depth) is not int or not 10 <= depth <= 45:
        raise ValueError("scratch depth must be an integer in [10, 45]")
    source = released["text_config"]
    if (source["hidden_size"], source["num_hidden_layers"]) != (RELEASED_WIDTH, RELEASED_DEPTH):
        raise ValueError("expected the released geometry (hidden 5120, 40 layers)")
    if engram_anchor_width is not None and not scale_engram:
        raise ValueError("a fixed Engram geometry requires scale_engram")
    text = copy.deepcopy(source)
    for name, (multiple, pow2) in CHANNEL_RULES.items():
        text[name] = scale_channel(source[name], width, multiple, pow2)
    if scale_engram:
        text.update(scaled_engram_geometry(source, width, anchor_width=engram_anchor_width))
    if study:
        if text.get("n_shared_experts", 1) != STUDY_SHARED_EXPERTS:
            raise ValueError("the scaling study requires the single shared expert of the released model")
        text.update(n_shared_experts=STUDY_SHARED_EXPERTS, moe_intermediate_size=STUDY_EXPERT_WIDTH,
                    num_experts_per_tok=routed_top_k(width, sweep=sweep))
    up = lambda layer: (layer * depth + RELEASED_DEPTH - 1) // RELEASED_DEPTH          # first layer of a region: ceiling
    text["num_hidden_layers"] = depth
    text["compress_ratios"] = [source["compress_ratios"][i * RELEASED_DEPTH // depth] for i in range(depth)]
    for name in ("kv_source_layer_ids", "index_source_layer_ids"):
        text[name] = sorted({up(layer) for layer in source[name]})
    text["engram_layer_ids"] = [layer * depth // RELEASED_DEPTH for layer in source["engram_layer_ids"]]
    text["candidate_source_layer_id"] = up(source["candidate_source_layer_id"])
    text.update(num_nextn_predict_layers=0, dspark_target_layer_ids=[], dspark_block_size=0, max_position_embeddings=16384,
                rope_scaling={"rope_type": "default"}, use_cache=False)
    return {"model_type": "deepseek_v41", "architectures": ["DeepseekV41ForCausalLM"], "dtype": "bfloat16", "text_config": text,
            "vision_config": {"model_type": "deepseek_v41_vision", "num_hidden_layers": 0}}


def to_model_config(text: dict, **overrides):
    """This framework's ``V41Config`` of a (scaled) ``text_config``; ``overrides`` replace single fields (a smaller
    vocabulary or expert count for a smoke run)."""
    from .deepseek_v41 import V41Config

    rope = text["qk_rope_head_dim"]
    fields = dict(n_layer=text["num_hidden_layers"], hidden_size=text["hidden_size"], n_heads=text["num_attention_heads"],
                  head_dim=text["head_dim"], rope_dim=rope, index_head_dim=text["index_head_dim"], index_rope_dim=min(rope, text["index_head_dim"]),
                  n_routed_experts=text["n_routed_experts"], n_shared_experts=text.get("n_shared_experts", 1),
                  experts_top_k=text["num_experts_per_tok"], moe_inter=text["moe_intermediate_size"],
                  sequence_len=min(4096, text.get("max_position_embeddings", 4096)))
    if "vocab_size" in text:
        fields["vocab_size"] = text["vocab_size"]
    fields.update(overrides)
    return V41Config(**fields)
