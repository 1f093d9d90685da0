"""Named single-hypothesis optimization recipes layered over the frozen speedrun contract
(src/archlab/optimizers/recipes.py:38-318).  Each recipe changes exactly the listed controls;
everything else stays at the baseline values of ``OptimizationRecipe``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

MARIN = "https://github.com/marin-community/marin/blob/main/docs/reports/agent-moe-experiments.md"
MODDED = "https://github.com/KellerJordan/modded-nanogpt"
MUONEQ = "https://github.com/marin-community/marin/issues/6066"


@dataclass(frozen=True)
class OptimizationRecipe:
    name: str
    summary: str
    sources: tuple[str, ...]
    model_overrides: dict[str, Any] = field(default_factory=dict)
    matrix_optimizer: str = "normuon"
    matrix_lr: float = 0.02
    unembedding_lr: float = 0.008
    embedding_lr: float = 0.3
    scalar_lr: float = 0.5
    gradient_clip: float = 0.0
    adam_update_every: int = 1
    cautious_adam_weight_decay: bool = False


_HB = {"matrix_init_recipe": "hyperball"}
_FULL = {"per_head_muon": False}
# name, summary, sources, model overrides, trainer controls
_TABLE: list[tuple[str, str, tuple[str, ...], dict, dict]] = [
    ("baseline", "Frozen per-head NorMuon comparison contract.", (MODDED,), {}, {}),
    ("full-matrix-muon", "One full Q/K/V matrix per layer instead of per-head optimizer partitions.", (MODDED,), _FULL, {}),
    ("full-matrix-clip01", "Full-matrix NorMuon with gradient clipping at 0.1.", (MODDED, MARIN), _FULL, {"gradient_clip": 0.1}),
    ("partial-rope", "Rotate half of every attention head; the other half stays stationary.", (MARIN, MODDED), {"rope_fraction": 0.5}, {}),
    ("partial-rope-25", "Rotate one quarter of every attention head.", (MARIN,), {"rope_fraction": 0.25}, {}),
    ("pko", "Partial key offset on every layer over the stationary half-head.", (MARIN, MODDED),
     {"rope_fraction": 0.5, "partial_key_offset": "all"}, {}),
    ("pko-last", "Partial key offset only in the final full-context layer.", (MARIN,),
     {"rope_fraction": 0.5, "partial_key_offset": "last"}, {}),
    ("embed-std1", "Unit-standard-deviation token embedding initialisation.", (MARIN,), {"embedding_init_std": 1.0}, {}),
    ("qk-gain", "Learnable per-head Q/K gain initialised to 1.2.", (MODDED,), {"learnable_qk_gain": True}, {}),
    ("cached-attention", "Reuse one attention input across the final three layers.", (MARIN,), {"cached_attention_layers": 3}, {}),
    ("midpoint-kv", "Upper layers read K/V from the midpoint residual.", (MARIN,), {"reuse_midpoint_kv": True}, {}),
    ("bf16-loss", "Logits and cross entropy in BF16.", (MARIN,), {"loss_fp32": False}, {}),
    ("asymmetric-logits", "Asymmetric sigmoid logit transform.", (MODDED,), {"logit_transform": "asymmetric"}, {}),
    *[(f"z-loss-{tag}", f"Final-logit z-loss at weight {w:g}.", (MARIN,), {"z_loss_weight": w}, {})
      for tag, w in (("1e-4", 1e-4), ("5e-6", 5e-6), ("1e-6", 1e-6), ("2e-6", 2e-6), ("1e-5", 1e-5), ("2e-5", 2e-5))],
    ("z-loss-5e-6-clip005", "z-loss 5e-6 with gradient clipping at 0.05.", (MARIN,), {"z_loss_weight": 5e-6}, {"gradient_clip": 0.05}),
    ("z-loss-5e-6-clip01", "z-loss 5e-6 with gradient clipping at 0.1.", (MARIN,), {"z_loss_weight": 5e-6}, {"gradient_clip": 0.1}),
    ("full-matrix-z-loss-5e-6-clip01", "Full-matrix NorMuon, z-loss 5e-6, clipping at 0.1.", (MARIN, MODDED),
     {**_FULL, "z_loss_weight": 5e-6}, {"gradient_clip": 0.1}),
    ("muonh", "NorMuon direction with a Frobenius-hyperball norm-preserving step.", (MODDED,), _HB, {"matrix_optimizer": "muonh"}),
    *[(f"muonh-lr{tag}", f"MuonH learning-rate retune at {lr:g}.", (MODDED,), _HB, {"matrix_optimizer": "muonh", "matrix_lr": lr})
      for tag, lr in (("01", 0.01), ("005", 0.005), ("03", 0.03), ("05", 0.05))],
    ("muonh-tuned-aux", "MuonH with the optimisation-track auxiliary learning-rate proportions.", (MODDED,), _HB,
     {"matrix_optimizer": "muonh", "matrix_lr": 0.018, "unembedding_lr": 0.00173, "embedding_lr": 0.246, "scalar_lr": 0.0195}),
    ("muoneqh-half", "MuonH with two-sided row/column equilibration exponent -1/2.", (MUONEQ,), _HB, {"matrix_optimizer": "muoneqh-half"}),
    ("muoneqh-quarter", "MuonH with equilibration exponent -1/4.", (MUONEQ,), _HB, {"matrix_optimizer": "muoneqh-quarter"}),
    ("adamh", "Adam-preconditioned Frobenius-hyperball updates for hidden matrices.", (MODDED,), _HB, {"matrix_optimizer": "adamh"}),
    *[(f"grad-clip-{tag}", f"Global gradient clipping at {c:g}.", (MARIN,), {}, {"gradient_clip": c})
      for tag, c in (("01", 0.1), ("005", 0.05), ("015", 0.15), ("02", 0.2), ("03", 0.3))],
    ("adam-every-2", "Auxiliary Adam parameters accumulate gradients and update every second step.", (MODDED,), {}, {"adam_update_every": 2}),
    ("cautious-adam-wd", "Auxiliary Adam weight decay only where update and parameter agree in sign.", (MODDED,), {},
     {"cautious_adam_weight_decay": True}),
    ("marin-compound", "Portable part of the combined-best recipe.", (MARIN,),
     {"rope_fraction": 0.5, "partial_key_offset": "all", "cached_attention_layers": 3, "embedding_init_std": 1.0}, {}),
]
OPTIMIZATION_RECIPES = {n: OptimizationRecipe(n, s, src, dict(mo), **ctl) for n, s, src, mo, ctl in _TABLE}


def get_optimization_recipe(name: str) -> OptimizationRecipe:
    try:
        return OPTIMIZATION_RECIPES[name]
    except KeyError as e:
        raise ValueError(f"unknown optimization recipe {name!r}; choose one of: {', '.join(OPTIMIZATION_RECIPES)}") from e
