"""Comparison regimes, artifact policy and training-budget resolution
(src/archlab/contracts.py:21-233)."""
from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass
from enum import Enum
from typing import Any


class ContractError(ValueError):
    pass


class ComparisonRegime(str, Enum):
    CONTROLLED = "controlled"
    FIXED_COMPUTE = "fixed_compute"
    SCALING = "scaling"


@dataclass(frozen=True)
class ComparisonContract:
    regime: ComparisonRegime
    baseline_variant: str = "baseline"
    paired_seed: bool = True
    paired_data_order: bool = True
    shared_initialization: str = "hash"
    primary_metric: str = "validation_bpb"

    @classmethod
    def from_mapping(cls, value: Mapping[str, Any]) -> "ComparisonContract":
        if "regime" not in value:
            raise ContractError("comparison.regime is required")
        try:
            regime = ComparisonRegime(str(value["regime"]))
        except ValueError as e:
            raise ContractError("comparison.regime must be one of: "
                                + ", ".join(r.value for r in ComparisonRegime)) from e
        c = cls(regime, str(value.get("baseline_variant", "baseline")), bool(value.get("paired_seed", True)),
                bool(value.get("paired_data_order", True)), str(value.get("shared_initialization", "hash")),
                str(value.get("primary_metric", "validation_bpb")))
        c.validate()
        return c

    def validate(self) -> None:
        if not self.baseline_variant:
            raise ContractError("comparison.baseline_variant must not be empty")
        if self.shared_initialization not in {"hash", "bit_identical", "not_applicable"}:
            raise ContractError("comparison.shared_initialization must be hash, bit_identical, or not_applicable")
        if not self.primary_metric:
            raise ContractError("comparison.primary_metric must not be empty")


@dataclass(frozen=True)
class ArtifactPolicy:
    mode: str = "research"
    save_final_checkpoint: bool = True
    save_optimizer_state: bool = True
    save_dataloader_state: bool = True
    raw_metrics: bool = True
    require_data_manifest: bool = True

    @classmethod
    def from_mapping(cls, value: Mapping[str, Any]) -> "ArtifactPolicy":
        p = cls(str(value.get("mode", "research")), *(bool(value.get(k, True)) for k in (
            "save_final_checkpoint", "save_optimizer_state", "save_dataloader_state", "raw_metrics",
            "require_data_manifest")))
        p.validate()
        return p

    def validate(self) -> None:
        if self.mode not in {"research", "metrics_only", "frozen_historical"}:
            raise ContractError("artifacts.mode must be research, metrics_only, or frozen_historical")
        if self.mode == "research" and not all((self.save_final_checkpoint, self.save_optimizer_state,
                                                self.save_dataloader_state, self.raw_metrics,
                                                self.require_data_manifest)):
            raise ContractError("research artifact policy may not disable required artifacts")


@dataclass(frozen=True)
class BudgetResolution:
    regime: ComparisonRegime
    steps: int
    effective_training_tokens: int
    requested_training_tokens: int | None
    requested_model_flops: float | None
    effective_model_flops: float | None
    tokens_per_parameter: float


def _pos_int(v, label: str) -> int:
    if v is None or v <= 0:
        raise ContractError(f"{label} must be a positive integer")
    return int(v)


def _pos_finite(v, label: str, regime: str) -> float:
    if v is None or not math.isfinite(v):
        raise ContractError(f"{label} must be finite for {regime}")
    if v <= 0:
        raise ContractError(f"{label} must be positive")
    return float(v)


def resolve_training_budget(regime, *, batch_tokens: int, parameter_count: int,
                            algorithmic_flops_per_token: float | None = None,
                            target_train_tokens: int | None = None, target_model_flops: float | None = None,
                            tokens_per_parameter: float | None = None) -> BudgetResolution:
    """Hard caps (controlled, fixed_compute) floor to whole steps; the tokens/parameter ratio of a
    scaling run rounds to the nearest step.  Mixing budget kinds is an error."""
    regime = ComparisonRegime(regime)
    batch_tokens = _pos_int(batch_tokens, "batch_tokens")
    parameter_count = _pos_int(parameter_count, "parameter_count")
    req_tokens = req_flops = None
    if regime is ComparisonRegime.CONTROLLED:
        req_tokens = _pos_int(target_train_tokens, "target_train_tokens")
        if target_model_flops is not None or tokens_per_parameter is not None:
            raise ContractError("controlled comparisons accept only target_train_tokens; do not mix budgets")
        steps = req_tokens // batch_tokens
    elif regime is ComparisonRegime.FIXED_COMPUTE:
        req_flops = _pos_finite(target_model_flops, "target_model_flops", "fixed_compute")
        fpt = _pos_finite(algorithmic_flops_per_token, "algorithmic_flops_per_token", "fixed_compute")
        if target_train_tokens is not None or tokens_per_parameter is not None:
            raise ContractError("fixed_compute comparisons accept only target_model_flops; do not mix budgets")
        steps = math.floor(req_flops / (fpt * batch_tokens))
    else:
        tpp = _pos_finite(tokens_per_parameter, "tokens_per_parameter", "scaling")
        if target_train_tokens is not None or target_model_flops is not None:
            raise ContractError("scaling comparisons accept only tokens_per_parameter; do not mix budgets")
        req_tokens = round(tpp * parameter_count)
        steps = round(req_tokens / batch_tokens)
    if steps < 1:
        raise ContractError("the resolved budget is smaller than one optimizer step")
    eff = steps * batch_tokens
    eff_flops = None if algorithmic_flops_per_token is None else float(algorithmic_flops_per_token) * eff
    return BudgetResolution(regime, steps, eff, req_tokens, req_flops, eff_flops, eff / parameter_count)


PAIRED_FIELDS = ("seed", "dataset_manifest_sha256", "tokenizer_sha256", "data_order_id", "training_tokens",
                 "sequence_length", "global_batch_tokens", "optimizer_contract_sha256")


def assert_paired_controls(baseline: Mapping[str, Any], variant: Mapping[str, Any], *,
                           fields: tuple[str, ...] = PAIRED_FIELDS) -> None:
    bad = {f: (baseline.get(f), variant.get(f)) for f in fields if baseline.get(f) != variant.get(f)}
    if bad:
        raise ContractError("controlled comparison mismatch: "
                            + ", ".join(f"{k}={a!r}/{b!r}" for k, (a, b) in bad.items()))
