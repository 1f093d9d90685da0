"""Result tables and curves from run receipts: paired comparisons against a baseline, smoothed learning
curves, markdown tables (src/archlab/reporting/paired_curves.py, learning_curves.py, runs.py)."""
from __future__ import annotations

import json
import math
from pathlib import Path
from statistics import mean, median


def read_metrics(path) -> list[dict]:
    out = []
    for line in Path(path).read_text().splitlines():
        if line.strip():
            out.append(json.loads(line))
    return out


def learning_curve(rows: list[dict], key: str = "loss", *, ema: float = 0.0) -> list[tuple[int, float]]:
    pts, acc = [], None
    for r in rows:
        if key not in r or not math.isfinite(r[key]):
            continue
        acc = r[key] if acc is None or ema <= 0 else ema * acc + (1 - ema) * r[key]
        pts.append((int(r.get("step", len(pts) + 1)), acc))
    return pts


def final_value(rows: list[dict], key: str = "loss", *, tail: int = 10) -> float:
    vals = [r[key] for r in rows if key in r and math.isfinite(r[key])][-tail:]
    if not vals:
        raise ValueError(f"no finite {key!r} values")
    return mean(vals)


def paired_comparison(runs: dict[str, dict[int, float]], baseline: str) -> list[dict]:
    """``runs[variant][seed] = metric`` (lower is better).  Differences are taken seed by seed against the
    baseline so shared data-order noise cancels."""
    if baseline not in runs:
        raise ValueError("baseline variant missing")
    rows = []
    for variant, by_seed in sorted(runs.items()):
        seeds = sorted(set(by_seed) & set(runs[baseline]))
        if not seeds:
            continue
        diffs = [by_seed[s] - runs[baseline][s] for s in seeds]
        sd = (sum((d - mean(diffs)) ** 2 for d in diffs) / (len(diffs) - 1)) ** 0.5 if len(diffs) > 1 else float("nan")
        rows.append({"variant": variant, "seeds": len(seeds), "mean": mean(by_seed[s] for s in seeds), "delta_mean": mean(diffs),
                     "delta_median": median(diffs), "delta_sd": sd,
                     "wins": sum(d < 0 for d in diffs), "losses": sum(d > 0 for d in diffs)})
    return rows


def markdown_table(rows: list[dict], columns: list[str], *, digits: int = 4) -> str:
    fmt = lambda v: f"{v:.{digits}f}" if isinstance(v, float) else str(v)
    head = "| " + " | ".join(columns) + " |\n|" + "|".join("---" for _ in columns) + "|\n"
    return head + "".join("| " + " | ".join(fmt(r.get(c, "")) for c in columns) + " |\n" for r in rows)
