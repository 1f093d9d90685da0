"""Integrity rules of a published metric table (CSV, one row per campaign x scale x variant).

Every row is checked against a small set of rules before a table is published or read back (the reference's checks:
src/archlab/results.py:22-82): required columns, no duplicate (campaign, scale, variant), a known status, finite positive
bits-per-byte where one is published, completed rows with all three seeds and a value, failed rows without one, positive
parameter counts and throughput ratios, ISO dates, and a paired delta that really is the row's value minus the
baseline of its campaign and scale.
"""
from __future__ import annotations

import csv
import math
from datetime import date
from pathlib import Path

REQUIRED = ("campaign", "scale", "budget_regime", "variant", "parameters", "mean_final_bpb", "paired_delta_bpb", "valid_seeds",
            "throughput_ratio", "status", "as_of")
STATUSES = ("complete", "partial", "failed-nonfinite")
SEEDS = 3


def load_table(path) -> list[dict[str, str]]:
    with Path(path).open(newline="", encoding="utf-8") as f:
        return list(csv.DictReader(f))


def _number(text: str, what: str, key) -> float:
    value = float(text)
    if not math.isfinite(value):
        raise ValueError(f"invalid {what} for {key}: {text}")
    return value


def verify_table(path) -> dict[str, int]:
    rows = load_table(path)
    if not rows or not set(REQUIRED) <= rows[0].keys():
        raise ValueError(f"metric table is missing required columns: {sorted(REQUIRED)}")
    baseline = {(r["campaign"], r["scale"]): float(r["mean_final_bpb"]) for r in rows if r["variant"] == "baseline" and r["mean_final_bpb"]}
    seen = set()
    for r in rows:
        key = (r["campaign"], r["scale"], r["variant"])
        if key in seen:
            raise ValueError(f"duplicate metric row: {key}")
        seen.add(key)
        status, bpb_text, seeds = r["status"], r["mean_final_bpb"], int(r["valid_seeds"])
        bpb = _number(bpb_text, "BPB", key) if bpb_text else None
        delta = _number(r["paired_delta_bpb"], "paired delta", key) if r["paired_delta_bpb"] else None
        rules = (
            (status not in STATUSES, f"unknown result status for {key}: {status}"),
            (status == "complete" and bpb is None, f"completed row has no BPB: {key}"),
            (bpb is not None and bpb <= 0, f"invalid BPB for {key}: {bpb_text}"),
            (not 0 <= seeds <= SEEDS, f"invalid seed count for {key}: {seeds}"),
            (status == "complete" and seeds != SEEDS, f"completed row must contain {SEEDS} seeds: {key}"),
            (status == "failed-nonfinite" and (bpb is not None or seeds != 0), f"failed row must not publish a BPB: {key}"),
            (bool(r["parameters"]) and int(r["parameters"]) <= 0, f"invalid parameter count for {key}"),
            (bool(r["throughput_ratio"]) and _number(r["throughput_ratio"] or "1", "throughput ratio", key) <= 0,
             f"invalid throughput ratio for {key}: {r['throughput_ratio']}"),
        )
        for violated, message in rules:
            if violated:
                raise ValueError(message)
        date.fromisoformat(r["as_of"])
        base = baseline.get(key[:2])
        if status == "complete" and None not in (base, bpb, delta) and not math.isclose(delta, bpb - base, abs_tol=2e-9):
            raise ValueError(f"paired delta disagrees with the published baseline for {key}")
    return {"rows": len(rows), "campaigns": len({r["campaign"] for r in rows})}
