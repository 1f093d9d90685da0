"""Comparing two training arms on what they can be compared on: speed over the SAME updates, and where one loss curve
overtakes the other for good.

``compare_throughput(baseline_dir, other_dir, first, last)`` reads both ``train.jsonl`` ledgers (uninterrupted fresh
runs: steps 1..n, finite measurements, positive denominators), requires that every common update saw the same step,
token counts and learning rate (otherwise the arms did not do the same work), and reports per-arm statistics over the
pre-declared window ``first..last`` (warm-up and compilation excluded by choosing ``first``), the ratio of total update
time, and a paired bootstrap interval over the window's steps -- variation among these steps, not run-to-run
uncertainty, and the report says so.  Both arms must start from the same held-out validation record.

``persistent_crossover`` gives the first step from which curve B stays below curve A for ``persistence`` consecutive
points (a single lucky point is not a crossover); ``trailing_mean`` is the causal smoother used before it.
(Reference: src/archlab/reporting/v41_attention_comparison.py:18-147, qwen38_early_curves.py:39-80.)
"""
from __future__ import annotations

import json
import math
import random
import statistics
from pathlib import Path

MATCHED_KEYS = ("step", "supervised_tokens", "input_tokens", "consumed_supervised_tokens", "learning_rate")


def read_fresh_ledger(path) -> list[dict]:
    rows = [json.loads(line) for line in Path(path).read_text().splitlines() if line.strip()]
    if [r["step"] for r in rows] != list(range(1, len(rows) + 1)):
        raise ValueError(f"expected an uninterrupted fresh-run ledger: {path}")
    for r in rows:
        if any(not math.isfinite(r[k]) for k in ("loss", "seconds", "gradient_norm_before_clip")):
            raise ValueError(f"non-finite training measurement: {path}")
        if r["seconds"] <= 0 or r["supervised_tokens"] <= 0:
            raise ValueError(f"invalid throughput denominator or token count: {path}")
    return rows


def percentile(values, fraction: float) -> float:
    v = sorted(values)
    pos = fraction * (len(v) - 1)
    lo, hi = math.floor(pos), math.ceil(pos)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


def window_statistics(rows: list[dict]) -> dict:
    seconds = [r["seconds"] for r in rows]
    targets, padded = sum(r["supervised_tokens"] for r in rows), sum(r.get("input_tokens", 0) for r in rows)
    out = {"steps": len(rows), "supervised_targets": targets, "padded_input_tokens": padded, "total_update_seconds": sum(seconds),
           "mean_update_seconds": statistics.mean(seconds), "median_update_seconds": statistics.median(seconds),
           "p10_update_seconds": percentile(seconds, 0.1), "p90_update_seconds": percentile(seconds, 0.9),
           "supervised_targets_per_second": targets / sum(seconds), "padded_input_tokens_per_second": padded / sum(seconds),
           "gradient_norm_range": [min(r["gradient_norm_before_clip"] for r in rows), max(r["gradient_norm_before_clip"] for r in rows)]}
    if all("max_memory_allocated_gib" in r for r in rows):
        out["peak_allocated_gib"] = max(r["max_memory_allocated_gib"] for r in rows)
    return out


def compare_throughput(baseline, other, *, first: int = 21, last: int = 50, draws: int = 10_000, seed: int = 2234) -> dict:
    if not 2 <= first <= last:
        raise ValueError("the comparison window must follow a logged earlier update")
    ledgers = [read_fresh_ledger(Path(d) / "train.jsonl") for d in (baseline, other)]
    if min(map(len, ledgers)) < last:
        raise ValueError(f"wait for the pre-declared step {last}; the ledgers hold {[len(l) for l in ledgers]}")
    for a, b in zip(*ledgers):
        for key in MATCHED_KEYS:
            if a.get(key) != b.get(key):
                raise ValueError(f"paired update {a['step']} differs in {key}")
    window = [l[first - 1:last] for l in ledgers]
    measured = [window_statistics(w) for w in window]
    ratio = measured[0]["total_update_seconds"] / measured[1]["total_update_seconds"]
    rng, n = random.Random(seed), last - first + 1
    resampled = []
    for _ in range(draws):
        idx = rng.choices(range(n), k=n)
        resampled.append(sum(window[0][i]["seconds"] for i in idx) / sum(window[1][i]["seconds"] for i in idx))
    validations = [[json.loads(line) for line in (Path(d) / "validation.jsonl").read_text().splitlines() if line.strip()] for d in (baseline, other)]
    if not validations[0] or not validations[1] or validations[0][0] != validations[1][0]:
        raise ValueError("the initial held-out validation of the two arms differs")
    return {"matched_steps": [first, last], "paired_update_count": n, "schedule_match_through_step": min(map(len, ledgers)),
            "baseline": measured[0], "other": measured[1], "throughput_ratio": ratio, "throughput_increase_percent": (ratio - 1) * 100,
            "update_time_reduction_percent": (1 - 1 / ratio) * 100,
            "paired_bootstrap_ratio_interval_95": [percentile(resampled, 0.025), percentile(resampled, 0.975)],
            "bootstrap_scope": "variation among these paired steps; not run-to-run uncertainty",
            "initial_validation": validations[1][0], "latest_other_validation": validations[1][-1]}


def trailing_mean(values: list[float], window: int) -> list[float]:
    out, total = [], 0.0
    for i, v in enumerate(values):
        total += v
        if i >= window:
            total -= values[i - window]
        out.append(total / min(i + 1, window))
    return out


def persistent_crossover(steps: list[int], a: list[float], b: list[float], *, persistence: int) -> int | None:
    """First step from which ``b < a`` holds for ``persistence`` consecutive points."""
    if not len(steps) == len(a) == len(b) or persistence < 1:
        raise ValueError("curves must be sampled at the same steps")
    below = [y < x for x, y in zip(a, b)]
    for i in range(len(below) - persistence + 1):
        if all(below[i:i + persistence]):
            return steps[i]
    return None


def median_step_seconds(events: list[tuple[int, float]], *, start_step: int, stop_step: int) -> float:
    """Median wall-clock spacing of logged events ``(step, wall time)`` inside a step range; NaN without two usable events."""
    picked = [e for e in events if start_step <= e[0] <= stop_step]
    gaps = [t1 - t0 for (_, t0), (_, t1) in zip(picked, picked[1:]) if t1 > t0]
    return statistics.median(gaps) if gaps else math.nan
