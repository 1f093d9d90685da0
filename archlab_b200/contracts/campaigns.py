"""Frozen parameter-scale campaigns: which architecture arms exist at which size, with the parameter
count, optimizer steps and warm-up that were fixed when the campaign was sealed, and the model
keyword arguments each arm adds to the shared geometry.

Same contract as the reference's campaign tables (src/archlab/campaigns.py:28-467): sixteen arms at
the 10M scale, the baseline at 100M (ClimbMix comparison, vocabulary 32768, 192 sequences of 2048
tokens per step), and parameter-free templates for the FineWeb scaling campaign (GPT-2 vocabulary
50304, five sizes) whose counts are resolved from the instantiated model.  The layout here is one
table of rows per campaign and one resolver; nothing is computed at import beyond indexing the rows.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

COMPARISON_SEEDS = (42, 43, 44)
COMPARISON_SEQUENCE_LENGTH = 2048
HISTORICAL_MICRO_BATCH_SIZE = 16
COMPARISON_GLOBAL_BATCH_SIZE = 192
COMPARISON_BATCH_TOKENS = COMPARISON_SEQUENCE_LENGTH * COMPARISON_GLOBAL_BATCH_SIZE
COMPARISON_EVAL_TOKENS = 3_932_160
FINEWEB_VOCAB_SIZE = 50_304
FINEWEB_TOKENS_PER_PARAMETER = 12.0
FINEWEB_FIXED_TOKEN_TARGETS = {"7b": 100_000_000_000}
TEN_M_SEEDS = COMPARISON_SEEDS

_SHARED = {"max_seq_len": COMPARISON_SEQUENCE_LENGTH, "window_pattern": "L", "fog_variant": "flash", "per_head_muon": True}


@dataclass(frozen=True)
class CampaignVariant:
    """One arm: its sealed size and schedule (zeros for a template) and the model arguments it adds."""

    name: str
    parameter_count: int
    steps: int
    warmup_steps: int
    model_overrides: tuple[tuple[str, Any], ...]

    @property
    def training_tokens(self) -> int:
        return self.steps * COMPARISON_BATCH_TOKENS

    def model_kwargs(self) -> dict[str, Any]:
        return dict(self.model_overrides)


TenMVariant = CampaignVariant

_SOTA = {"arch_family": "sota_pool", "sota_extra_lr": 0.005, "canon_kernel_size": 4, "bov_target_fraction": 1.0 / 3.0}
_FRONTIER = {"arch_family": "frontier_pool", "relative_dim": 8}
_KDA = {"arch_family": "kimi_kda", "kda_pattern": "KKKG", "kda_force_final_global": True}

# name, parameters, steps, warm-up, model arguments (10M geometry: depth 5, aspect ratio 11, head dim 8)
_TEN_M_ROWS: tuple[tuple[str, int, int, int, dict[str, Any]], ...] = (
    ("baseline", 9_363_488, 286, 14, {**_SOTA, "sota_variant": "baseline"}),
    ("engram", 10_284_800, 314, 16, {"arch_family": "engram", "engram_ngram_orders": (2, 3), "engram_kernel_size": 4,
                                     "engram_seed": 0, "engram_layers": (2,), "engram_num_heads": 2, "engram_dim": 28,
                                     "engram_vocab_multiplier": 1}),
    ("kda", 9_372_437, 286, 14, {**_KDA, "kda_rope_policy": "global_only", "kda_variant": "kimi_linear"}),
    ("dsa", 9_391_248, 287, 14, {"arch_family": "deepseek_dsa", "dsa_top_k": 32, "dsa_query_chunk_size": 128,
                                 "dsa_backend": "sdpa_masked", "dsa_warmup_indexer_lr": 1e-3,
                                 "dsa_sparse_indexer_lr": 7.3e-6, "dsa_index_heads": 2, "dsa_index_head_dim": 32,
                                 "dsa_index_rope_dim": 8}),
    ("attnres", 9_364_709, 286, 14, {"arch_family": "kimi_attnres", "attn_res_block_size": 2, "attn_res_recompute": True,
                                     "attn_res_variant": "kimi_k3_block_attnres", "attn_res_heads": 1}),
    ("mhc", 9_417_518, 287, 14, {"arch_family": "mhc"}),
    ("gated-attention", 9_365_448, 286, 14, {**_SOTA, "sota_variant": "gated_attention"}),
    ("situ-glu", 9_363_208, 286, 14, {**_FRONTIER, "frontier_variant": "kimi_situ_glu"}),
    ("inkling-relative-attention", 9_420_128, 287, 14, {**_FRONTIER, "frontier_variant": "inkling_relative_attention"}),
    ("glm-mla", 9_394_848, 287, 14, {**_FRONTIER, "frontier_variant": "glm_mla_muon_split"}),
    ("xielu", 9_363_498, 286, 14, {**_SOTA, "sota_variant": "xielu"}),
    ("qwen-gdn", 9_423_916, 288, 14, {**_FRONTIER, "frontier_variant": "qwen_gdn"}),
    ("inkling-sconv-kv", 9_365_728, 286, 14, {**_FRONTIER, "frontier_variant": "inkling_sconv_kv"}),
    ("inkling-sconv-residual", 9_365_728, 286, 14, {**_FRONTIER, "frontier_variant": "inkling_sconv_residual"}),
    ("partial-rope-25", 9_363_488, 286, 14, {**_FRONTIER, "frontier_variant": "partial_rope_25"}),
    ("kimi-k3-kda-update", 9_385_429, 286, 14, {**_KDA, "kda_variant": "kimi_k3", "kda_rope_policy": "none"}),
)
_HUNDRED_M_ROWS = (("baseline", 105_775_510, 3_228, 40, {**_SOTA, "sota_variant": "baseline"}),)


def _arms(rows) -> tuple[CampaignVariant, ...]:
    return tuple(CampaignVariant(n, p, s, w, tuple(kw.items())) for n, p, s, w, kw in rows)


TEN_M_VARIANTS = _arms(_TEN_M_ROWS)
HUNDRED_M_VARIANTS = _arms(_HUNDRED_M_ROWS)
TEN_M_VARIANTS_BY_NAME = {v.name: v for v in TEN_M_VARIANTS}
HUNDRED_M_VARIANTS_BY_NAME = {v.name: v for v in HUNDRED_M_VARIANTS}
CAMPAIGN_GEOMETRIES = {"10m": {"depth": 5, "aspect_ratio": 11, "head_dim": 8},
                       "100m": {"depth": 10, "aspect_ratio": 38, "head_dim": 64}}
CAMPAIGN_VARIANTS = {"10m": TEN_M_VARIANTS_BY_NAME, "100m": HUNDRED_M_VARIANTS_BY_NAME}

# FineWeb scaling campaign: widths chosen so that the baseline lands near the nominal label with the larger
# vocabulary (which also widens the value-embedding bank); 32 x 3200 at "7b" resolves to 6.83B parameters.
FINEWEB_CAMPAIGN_GEOMETRIES = {
    "1m": {"depth": 2, "aspect_ratio": 4, "head_dim": 8},
    "10m": {"depth": 5, "aspect_ratio": 7, "head_dim": 8},
    "100m": {"depth": 10, "aspect_ratio": 20, "head_dim": 64},
    "300m": {"depth": 16, "aspect_ratio": 29, "head_dim": 64},
    "7b": {"depth": 32, "aspect_ratio": 100, "head_dim": 128},
}
# per size: (engram layers, engram heads, engram dim), (indexer heads, head dim, rope dim), relative dim
_FINEWEB_CONTROLS = {
    "1m": (((0,), 1, 2), (1, 8, 4), 4),
    "10m": (((2,), 2, 20), (2, 32, 8), 8),
    "100m": (((1, 4), 4, 128), (4, 64, 32), 16),
    "300m": (((3, 9), 8, 256), (8, 64, 32), 32),
    "7b": (((7, 15, 23, 31), 16, 512), (16, 128, 64), 64),
}


def _fineweb_arm(scale: str, base: CampaignVariant) -> CampaignVariant:
    kw = base.model_kwargs()
    engram, dsa, rel = _FINEWEB_CONTROLS[scale]
    if base.name == "engram":
        kw.update(zip(("engram_layers", "engram_num_heads", "engram_dim"), engram))
    elif base.name == "dsa":
        kw.update(zip(("dsa_index_heads", "dsa_index_head_dim", "dsa_index_rope_dim"), dsa))
    elif kw.get("arch_family") == "frontier_pool":
        kw["relative_dim"] = rel
    return CampaignVariant(base.name, 0, 0, 0, tuple(kw.items()))


_COLU = CampaignVariant("colu", 0, 0, 0, tuple({"arch_family": "combo_search", "search_mlp": "colu", "colu_dim": 4}.items()))
FINEWEB_CAMPAIGN_VARIANTS = {scale: {**{b.name: _fineweb_arm(scale, b) for b in TEN_M_VARIANTS}, "colu": _COLU}
                             for scale in FINEWEB_CAMPAIGN_GEOMETRIES}


def _pick(table: dict, key: str, what: str):
    if key not in table:
        raise ValueError(f"unknown {what} {key!r}; choose one of: {', '.join(table)}")
    return table[key]


def get_ten_m_variant(name: str) -> CampaignVariant:
    return _pick(TEN_M_VARIANTS_BY_NAME, name, "10M variant")


def get_campaign_variant(scale: str, name: str) -> CampaignVariant:
    return _pick(_pick(CAMPAIGN_VARIANTS, scale, "campaign scale"), name, f"{scale} variant")


def get_fineweb_variant_template(scale: str, name: str) -> CampaignVariant:
    return _pick(_pick(FINEWEB_CAMPAIGN_VARIANTS, scale, "FineWeb scale"), name, f"FineWeb {scale} variant")


def campaign_model_config_kwargs(scale: str, variant: CampaignVariant) -> dict[str, Any]:
    """Shared geometry of the ClimbMix comparison at ``scale`` plus the arm's mechanism."""
    return {**_pick(CAMPAIGN_GEOMETRIES, scale, "campaign scale"), **_SHARED, "vocab_size": 32_768, **variant.model_kwargs()}


def ten_m_model_config_kwargs(variant: CampaignVariant) -> dict[str, Any]:
    return campaign_model_config_kwargs("10m", variant)


def fineweb_model_config_kwargs(scale: str, variant: CampaignVariant) -> dict[str, Any]:
    """GPT-2-vocabulary geometry of the FineWeb campaign at ``scale`` plus the arm's mechanism."""
    return {**_pick(FINEWEB_CAMPAIGN_GEOMETRIES, scale, "FineWeb scale"), **_SHARED, "vocab_size": FINEWEB_VOCAB_SIZE,
            **variant.model_kwargs()}


def fineweb_token_budget(scale: str, parameter_count: int) -> int:
    """Tokens to train a resolved FineWeb arm on: the fixed target of the size if it has one, else 12 per parameter."""
    _pick(FINEWEB_CAMPAIGN_GEOMETRIES, scale, "FineWeb scale")
    return FINEWEB_FIXED_TOKEN_TARGETS.get(scale, int(round(FINEWEB_TOKENS_PER_PARAMETER * parameter_count)))


def verify_ten_m_contract() -> dict[str, int]:
    names = [v.name for v in TEN_M_VARIANTS]
    if len(names) != 16 or len(set(names)) != 16:
        raise RuntimeError("the 10M campaign must contain 16 unique variants")
    if any(v.training_tokens <= 0 for v in TEN_M_VARIANTS):
        raise RuntimeError("the 10M campaign contains an invalid token budget")
    return {"variants": len(names), "seeds": len(TEN_M_SEEDS), "runs": len(names) * len(TEN_M_SEEDS)}
