"""Aggregating the frozen 10M campaign (16 variants x seeds) and asking whether two execution backends AGREE on which
variants help.

A campaign row is one finished run ``(backend, variant, seed)`` with its sealed size and schedule, final bits per byte
and throughput.  Rows come from ``result.json`` receipts under a results tree or from a CSV table (a published
reference).  The rules:

* ``overlay`` replaces explicitly re-run keys and refuses keys the campaign never had; ``merge_recoveries`` fills missing
  keys and refuses to replace an existing row: a correction and a recovery cannot be confused with each other.
* ``validate`` checks every row against the campaign contract (parameter count, steps, tokens of its variant; known
  seeds; finite positive metrics) and, unless partial results are allowed, that every backend has every (variant, seed).
* ``summarize`` pairs each run with the SAME-SEED baseline of its backend: paired bpb delta, throughput normalised to
  the baseline, using steady-state throughput when every pair has it.
* ``cross_backend`` compares two backends' per-variant deltas: Pearson correlation, sign agreement, mean gaps, baseline
  gap and absolute throughput ratio.
(Reference: src/archlab/speedrun/campaign_compare.py:28-330.)
"""
from __future__ import annotations

import csv
import json
import math
import statistics
from collections import defaultdict
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Iterable

from ..contracts.campaigns import TEN_M_SEEDS, TEN_M_VARIANTS_BY_NAME


@dataclass(frozen=True)
class RunResult:
    backend: str
    variant: str
    seed: int
    parameter_count: int
    training_steps: int
    training_tokens: int
    final_bpb: float
    tokens_per_second: float
    wall_seconds: float
    source_commit: str = ""
    optimization_recipe: str = ""
    steady_state_tokens_per_second: float | None = None

    @property
    def key(self) -> tuple[str, str, int]:
        return self.backend, self.variant, self.seed


def _name(field) -> str:
    return field.get("name", "") if isinstance(field, dict) else str(field or "")


def load_results(root, backend: str) -> list[RunResult]:
    rows = []
    for path in sorted(Path(root).rglob("result.json")):
        body = json.loads(path.read_text())
        if body.get("backend") != backend or body.get("mode", "full") != "full":
            continue
        steady = body.get("steady_state_tokens_per_second")
        rows.append(RunResult(backend, _name(body["variant"]), int(body["seed"]), int(body["parameter_count"]), int(body["training_steps"]),
                              int(body["training_tokens"]), float(body["final_bpb"]), float(body["tokens_per_second"]), float(body["wall_seconds"]),
                              str(body.get("source_commit", "")), _name(body.get("optimization_recipe")), None if steady is None else float(steady)))
    return rows


def load_table(path) -> list[RunResult]:
    with Path(path).open(newline="") as f:
        rows = []
        for r in csv.DictReader(f):
            steady = r.get("steady_state_tokens_per_second") or None
            rows.append(RunResult(r["backend"], r["variant"], int(r["seed"]), int(r["parameter_count"]), int(r["training_steps"]), int(r["training_tokens"]),
                                  float(r["final_bpb"]), float(r["tokens_per_second"]), float(r["wall_seconds"]), r.get("source_commit", ""),
                                  r.get("optimization_recipe", ""), None if steady is None else float(steady)))
        return rows


def _indexed(rows, what: str) -> dict:
    rows = list(rows)
    table = {r.key: r for r in rows}
    if len(table) != len(rows):
        raise ValueError(f"{what} contains duplicate rows")
    return table


def overlay(primary: Iterable[RunResult], corrections: Iterable[RunResult]) -> list[RunResult]:
    table, fixes = _indexed(primary, "the primary campaign"), _indexed(corrections, "the correction overlay")
    unknown = sorted(set(fixes) - set(table))
    if unknown:
        raise ValueError(f"the correction overlay contains unknown rows: {unknown[:5]}")
    return sorted({**table, **fixes}.values(), key=lambda r: r.key)


def merge_recoveries(primary: Iterable[RunResult], recoveries: Iterable[RunResult]) -> list[RunResult]:
    table, extra = _indexed(primary, "the primary campaign"), _indexed(recoveries, "the recovery results")
    clash = sorted(set(extra) & set(table))
    if clash:
        raise ValueError(f"recovery results would replace existing rows: {clash[:5]}")
    return sorted({**table, **extra}.values(), key=lambda r: r.key)


def validate(rows: Iterable[RunResult], *, allow_partial: bool = False) -> list[RunResult]:
    rows = list(_indexed(rows, "the campaign").values())
    for r in rows:
        if r.variant not in TEN_M_VARIANTS_BY_NAME or r.seed not in TEN_M_SEEDS:
            raise ValueError(f"unexpected campaign row: {r.key}")
        c = TEN_M_VARIANTS_BY_NAME[r.variant]
        if (r.parameter_count, r.training_steps, r.training_tokens) != (c.parameter_count, c.steps, c.training_tokens):
            raise ValueError(f"contract drift for {r.key}")
        for name in ("final_bpb", "tokens_per_second"):
            if not math.isfinite(getattr(r, name)) or getattr(r, name) <= 0:
                raise ValueError(f"invalid {name} for {r.key}")
    if not allow_partial:
        want = {(v, s) for v in TEN_M_VARIANTS_BY_NAME for s in TEN_M_SEEDS}
        for backend in {r.backend for r in rows}:
            missing = sorted(want - {(r.variant, r.seed) for r in rows if r.backend == backend})
            if missing:
                raise ValueError(f"{backend} is missing {len(missing)} frozen runs: {missing[:5]}")
    return rows


def summarize(rows: Iterable[RunResult]) -> list[dict]:
    groups, baselines = defaultdict(list), {}
    for r in rows:
        groups[(r.backend, r.variant)].append(r)
        if r.variant == "baseline":
            baselines[(r.backend, r.seed)] = r
    out = []
    for (backend, variant), members in sorted(groups.items()):
        pairs = [(r, baselines[(backend, r.seed)]) for r in members if (backend, r.seed) in baselines]
        if not pairs:
            continue
        steady = all(r.steady_state_tokens_per_second is not None and b.steady_state_tokens_per_second is not None for r, b in pairs)
        speed = (lambda r: r.steady_state_tokens_per_second) if steady else (lambda r: r.tokens_per_second)
        out.append({"backend": backend, "variant": variant, "seeds": len(pairs), "mean_bpb": statistics.fmean(r.final_bpb for r, _ in pairs),
                    "paired_delta_bpb": statistics.fmean(r.final_bpb - b.final_bpb for r, b in pairs),
                    "mean_tokens_per_second": statistics.fmean(speed(r) for r, _ in pairs),
                    "normalized_throughput": statistics.fmean(speed(r) / speed(b) for r, b in pairs),
                    "mean_wall_seconds": statistics.fmean(r.wall_seconds for r, _ in pairs),
                    "throughput_basis": "median steady-state step" if steady else "aggregate after warm-up"})
    return out


def pearson(x: list[float], y: list[float]) -> float:
    if len(x) != len(y) or len(x) < 2:
        return float("nan")
    mx, my = statistics.fmean(x), statistics.fmean(y)
    den = math.sqrt(sum((a - mx) ** 2 for a in x) * sum((b - my) ** 2 for b in y))
    return sum((a - mx) * (b - my) for a, b in zip(x, y)) / den if den else float("nan")


def cross_backend(summaries: list[dict], first: str, second: str) -> dict:
    table = {(s["backend"], s["variant"]): s for s in summaries}
    variants = sorted(v for v in TEN_M_VARIANTS_BY_NAME if v != "baseline" and (first, v) in table and (second, v) in table)
    a = [table[(first, v)]["paired_delta_bpb"] for v in variants]
    b = [table[(second, v)]["paired_delta_bpb"] for v in variants]
    gaps = [y - x for x, y in zip(a, b)]
    agree = sum((x < 0) == (y < 0) for x, y in zip(a, b))
    out = {"variants": variants, "variant_count": len(variants), "delta_pearson": pearson(a, b),
           "mean_absolute_delta_gap": statistics.fmean(map(abs, gaps)) if gaps else None, "mean_signed_delta_gap": statistics.fmean(gaps) if gaps else None,
           "delta_sign_agreement_count": agree, "delta_sign_agreement_rate": agree / len(variants) if variants else None}
    if (first, "baseline") in table and (second, "baseline") in table:
        out["baseline_bpb_gap"] = table[(second, "baseline")]["mean_bpb"] - table[(first, "baseline")]["mean_bpb"]
        out["baseline_absolute_throughput_ratio"] = table[(second, "baseline")]["mean_tokens_per_second"] / table[(first, "baseline")]["mean_tokens_per_second"]
    return out


def write_comparison(output, rows: list[RunResult], first: str, second: str) -> dict:
    output = Path(output)
    output.mkdir(parents=True, exist_ok=True)
    summaries = summarize(rows)
    metrics = cross_backend(summaries, first, second)
    with (output / "runs.csv").open("w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(asdict(rows[0])))
        w.writeheader()
        w.writerows(asdict(r) for r in rows)
    with (output / "variants.csv").open("w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(summaries[0]))
        w.writeheader()
        w.writerows(summaries)
    lines = ["| variant | " + " | ".join(f"{b} delta bpb | {b} rel. throughput" for b in (first, second)) + " |", "|---|" + "---|" * 4]
    table = {(s["backend"], s["variant"]): s for s in summaries}
    for v in ["baseline", *metrics["variants"]]:
        cells = []
        for b in (first, second):
            s = table.get((b, v))
            cells += ["-", "-"] if s is None else [f"{s['paired_delta_bpb']:+.4f}", f"{s['normalized_throughput']:.3f}"]
        lines.append(f"| {v} | " + " | ".join(cells) + " |")
    (output / "comparison.md").write_text("\n".join(lines) + "\n\n" + json.dumps({k: v for k, v in metrics.items() if k != "variants"}, indent=1) + "\n")
    (output / "comparison.json").write_text(json.dumps({"metrics": metrics, "summaries": summaries}, indent=1) + "\n")
    return metrics
