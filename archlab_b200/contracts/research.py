"""Research contracts: which question a comparison answers, what a reportable run must keep, and how a declared
budget becomes a whole number of optimizer steps.

Behaviour is that of the reference's contracts (src/archlab/contracts.py:17-262): three regimes (``controlled``,
``fixed_compute``, ``scaling``), each accepting exactly one budget quantity; hard budgets round down, the
tokens-per-parameter ratio rounds to the nearest step; a ``research`` artifact policy may switch nothing off; a
controlled pair must agree on every frozen axis.

The contracts parse through their own dataclass field tables, and each regime is one ``_BudgetRule`` row (the
quantity it accepts and how that quantity becomes steps), so the mixing check and the rounding rules are data.
"""
from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass, fields
from enum import Enum
from typing import Any, Callable


class ContractError(ValueError):
    """A comparison contract is incomplete or contradicts itself."""


class ComparisonRegime(str, Enum):
    CONTROLLED = "controlled"
    FIXED_COMPUTE = "fixed_compute"
    SCALING = "scaling"


INITIALIZATION_MODES = ("hash", "bit_identical", "not_applicable")
ARTIFACT_MODES = ("research", "metrics_only", "frozen_historical")


@dataclass(frozen=True)
class ComparisonContract:
    """What makes a baseline / variant pair interpretable."""
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
        except ValueError:
            raise ContractError("comparison.regime must be one of: " + ", ".join(r.value for r in ComparisonRegime)) from None
        rest = {k: v for k, v in value.items() if k != "regime"}
        typed = {"baseline_variant": str, "paired_seed": bool, "paired_data_order": bool, "shared_initialization": str,
                 "primary_metric": str}
        made = cls(regime, **{k: typed[k](v) for k, v in rest.items() if k in typed})
        made.validate()
        return made

    def validate(self) -> None:
        for name in ("baseline_variant", "primary_metric"):
            if not getattr(self, name):
                raise ContractError(f"comparison.{name} must not be empty")
        if self.shared_initialization not in INITIALIZATION_MODES:
            raise ContractError("comparison.shared_initialization must be " + ", ".join(INITIALIZATION_MODES[:-1])
                                + f", or {INITIALIZATION_MODES[-1]}")


@dataclass(frozen=True)
class ArtifactPolicy:
    """What a reportable run keeps on disk."""
    mode: str = "research"
    save_final_checkpoint: bool = True
    save_optimizer_state: bool = True
    save_dataloader_state: bool = True
    raw_metrics: bool = True
    require_data_manifest: bool = True

    @classmethod
    def from_mapping(cls, value: Mapping[str, Any]) -> "ArtifactPolicy":
        known = {f.name: (str if f.name == "mode" else bool) for f in fields(cls)}
        made = cls(**{k: known[k](v) for k, v in value.items() if k in known})
        made.validate()
        return made

    def switches(self) -> dict[str, bool]:
        return {f.name: getattr(self, f.name) for f in fields(self) if f.name != "mode"}

    def validate(self) -> None:
        if self.mode not in ARTIFACT_MODES:
            raise ContractError("artifacts.mode must be " + ", ".join(ARTIFACT_MODES[:-1]) + f", or {ARTIFACT_MODES[-1]}")
        off = [name for name, on in self.switches().items() if not on]
        if self.mode == "research" and off:
            raise ContractError(f"research artifact policy may not disable required artifacts ({', '.join(off)})")


@dataclass(frozen=True)
class BudgetResolution:
    """A whole number of optimizer steps derived from one declared budget."""
    regime: ComparisonRegime
    steps: int
    effective_training_tokens: int
    requested_training_tokens: int | None
    requested_model_flops: float | None
    effective_model_flops: float | None
    tokens_per_parameter: float


def _positive_finite(value, label: str, regime: str) -> float:
    if value is None or not math.isfinite(value):
        raise ContractError(f"{label} must be finite for {regime}")
    if value <= 0:
        raise ContractError(f"{label} must be positive")
    return float(value)


def _positive_int(value, label: str) -> int:
    if value is None or value <= 0:
        raise ContractError(f"{label} must be a positive integer")
    return int(value)


@dataclass(frozen=True)
class _BudgetRule:
    quantity: str                                              # the one budget argument this regime accepts
    steps: Callable[[dict], tuple[int, int | None, float | None]]   # -> (steps, requested tokens, requested flops)


def _controlled(a):
    tokens = _positive_int(a["target_train_tokens"], "target_train_tokens")
    return tokens // a["batch_tokens"], tokens, None            # a hard cap: round down


def _fixed_compute(a):
    flops = _positive_finite(a["target_model_flops"], "target_model_flops", "fixed_compute")
    per_token = _positive_finite(a["algorithmic_flops_per_token"], "algorithmic_flops_per_token", "fixed_compute")
    return math.floor(flops / (per_token * a["batch_tokens"])), None, flops   # a hard cap: round down


def _scaling(a):
    ratio = _positive_finite(a["tokens_per_parameter"], "tokens_per_parameter", "scaling")
    tokens = round(ratio * a["parameter_count"])
    return round(tokens / a["batch_tokens"]), tokens, None      # a ratio, not a cap: nearest step


_BUDGET_QUANTITIES = ("target_train_tokens", "target_model_flops", "tokens_per_parameter")
_BUDGET_RULES = {
    ComparisonRegime.CONTROLLED: _BudgetRule("target_train_tokens", _controlled),
    ComparisonRegime.FIXED_COMPUTE: _BudgetRule("target_model_flops", _fixed_compute),
    ComparisonRegime.SCALING: _BudgetRule("tokens_per_parameter", _scaling),
}


def resolve_training_budget(regime, *, batch_tokens: int, parameter_count: int, algorithmic_flops_per_token: float | None = None,
                            target_train_tokens: int | None = None, target_model_flops: float | None = None,
                            tokens_per_parameter: float | None = None) -> BudgetResolution:
    """Turns the regime's one budget quantity into optimizer steps; naming a second quantity is an error, because
    it would silently change the question the comparison answers."""
    regime = ComparisonRegime(regime)
    args = {"batch_tokens": _positive_int(batch_tokens, "batch_tokens"),
            "parameter_count": _positive_int(parameter_count, "parameter_count"),
            "algorithmic_flops_per_token": algorithmic_flops_per_token, "target_train_tokens": target_train_tokens,
            "target_model_flops": target_model_flops, "tokens_per_parameter": tokens_per_parameter}
    rule = _BUDGET_RULES[regime]
    steps, want_tokens, want_flops = rule.steps(args)
    if any(args[q] is not None for q in _BUDGET_QUANTITIES if q != rule.quantity):
        raise ContractError(f"{regime.value} comparisons accept only {rule.quantity}; do not mix budgets")
    if steps < 1:
        raise ContractError("the resolved budget is smaller than one optimizer step")
    tokens = steps * args["batch_tokens"]
    per_token = algorithmic_flops_per_token
    return BudgetResolution(regime, steps, tokens, want_tokens, want_flops,
                            None if per_token is None else float(per_token) * tokens, tokens / args["parameter_count"])


FROZEN_AXES = ("seed", "dataset_manifest_sha256", "tokenizer_sha256", "data_order_id", "training_tokens", "sequence_length",
               "global_batch_tokens", "optimizer_contract_sha256")


def assert_paired_controls(baseline: Mapping[str, Any], variant: Mapping[str, Any], *, fields: tuple[str, ...] = FROZEN_AXES) -> None:
    """A controlled comparison holds every frozen axis equal between baseline and variant."""
    differing = [f"{axis}={baseline.get(axis)!r}/{variant.get(axis)!r}" for axis in fields
                 if baseline.get(axis) != variant.get(axis)]
    if differing:
        raise ContractError("controlled comparison mismatch: " + ", ".join(differing))
