"""Throughput protocols and regression contracts.

``ThroughputProtocol`` / ``summarize_step_timestamps`` are the pre-training protocol (median step
after a warm-up window; src/archlab/performance.py:15-94).  ``ThroughputContract`` /
``check_throughput`` compare two ``throughput.json`` receipts taken under an identical contract
(src/archlab/training/performance.py:11-65).
"""
from __future__ import annotations

import json
import math
import statistics
from collections.abc import Sequence
from dataclasses import asdict, dataclass
from pathlib import Path


class PerformanceError(ValueError):
    pass


@dataclass(frozen=True)
class ThroughputProtocol:
    warmup_steps: int = 10
    measurement_steps: int = 0        # 0 = every remaining interval
    statistic: str = "median"

    def validate(self) -> None:
        if self.warmup_steps < 0 or self.measurement_steps < 0:
            raise PerformanceError("throughput step counts must be non-negative")
        if self.statistic != "median":
            raise PerformanceError("only the robust median throughput statistic is supported")

    def to_dict(self) -> dict:
        self.validate()
        return asdict(self)


def _empty(protocol: ThroughputProtocol) -> dict:
    return {"measured_training_seconds": 0.0, "tokens_per_second": 0.0, "median_step_seconds": 0.0,
            "p90_step_seconds": 0.0, "steady_state_tokens_per_second": 0.0, "throughput_sample_intervals": 0,
            "throughput_protocol": protocol.to_dict()}


def summarize_step_timestamps(timestamps: Sequence[float], *, tokens_per_step: int,
                              protocol: ThroughputProtocol | None = None) -> dict:
    """Timestamps are taken after each optimizer step; interval i lies between stamps i and i+1."""
    protocol = protocol or ThroughputProtocol()
    protocol.validate()
    if tokens_per_step <= 0:
        raise PerformanceError("tokens_per_step must be positive")
    if len(timestamps) < 2:
        return _empty(protocol)
    iv = [b - a for a, b in zip(timestamps[:-1], timestamps[1:])]
    if any(not math.isfinite(v) or v <= 0 for v in iv):
        raise PerformanceError("step timestamps must be finite and strictly increasing")
    start = min(protocol.warmup_steps, len(iv))
    stop = len(iv) if not protocol.measurement_steps else min(len(iv), start + protocol.measurement_steps)
    sel = iv[start:stop]
    if not sel:
        return _empty(protocol)
    ordered = sorted(sel)
    med = statistics.median(sel)
    return {"measured_training_seconds": sum(sel), "tokens_per_second": len(sel) * tokens_per_step / sum(sel),
            "median_step_seconds": med, "p90_step_seconds": ordered[max(0, math.ceil(0.9 * len(ordered)) - 1)],
            "steady_state_tokens_per_second": tokens_per_step / med, "throughput_sample_intervals": len(sel),
            "throughput_protocol": protocol.to_dict()}


@dataclass
class ThroughputContract:
    baseline: str = ""                 # path of the baseline receipt
    sequence_length: int = 2048
    warmup: int = 2
    samples: int = 5
    max_slowdown: float = 1.2

    def validate(self) -> None:
        if self.sequence_length < 1 or self.warmup < 0 or self.samples < 3:
            raise PerformanceError("throughput contract needs sequence_length >= 1, warmup >= 0, samples >= 3")
        if not (self.max_slowdown >= 1.0 and math.isfinite(self.max_slowdown)):
            raise PerformanceError("max_slowdown must be a finite ratio >= 1")

    def identity(self) -> dict:
        return {"sequence_length": self.sequence_length, "warmup": self.warmup, "samples": self.samples}


def throughput_receipt(contract: ThroughputContract, update_seconds: Sequence[float], **extra) -> dict:
    contract.validate()
    if len(update_seconds) != contract.samples:
        raise PerformanceError("receipt must hold exactly the contracted number of samples")
    return {"contract": contract.identity(), "update_seconds": list(map(float, update_seconds)),
            "median_update_seconds": statistics.median(update_seconds), **extra}


def check_throughput(contract: ThroughputContract, candidate: dict | str | Path,
                     baseline: dict | str | Path | None = None) -> dict:
    """Median-ratio gate between two receipts taken under the same contract."""
    contract.validate()

    def load(x):
        return json.loads(Path(x).read_text()) if isinstance(x, (str, Path)) else x

    cand = load(candidate)
    base = load(baseline if baseline is not None else contract.baseline)
    for name, r in (("candidate", cand), ("baseline", base)):
        if r.get("contract") != contract.identity():
            raise PerformanceError(f"{name} receipt was measured under a different contract")
        if len(r.get("update_seconds", [])) != contract.samples:
            raise PerformanceError(f"{name} receipt has the wrong number of samples")
    ratio = statistics.median(cand["update_seconds"]) / statistics.median(base["update_seconds"])
    return {"passed": ratio <= contract.max_slowdown, "slowdown": ratio, "max_slowdown": contract.max_slowdown,
            "candidate_median": statistics.median(cand["update_seconds"]),
            "baseline_median": statistics.median(base["update_seconds"])}
