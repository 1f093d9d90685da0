"""Reading the repeated-data sweep: only cells that finished exactly on budget count, comparisons are made at EQUAL
measured compute, and the loop frontier is a lower convex envelope -- never an extrapolation.

* ``load_measurements(plan)``: the plan must be the whole preregistered grid.  Every validation row with consumed tokens
  becomes a trajectory point (finite loss, positive training GPU-seconds); a cell enters the final comparison only with
  a ``COMPLETE.json`` that passed, consumed exactly the registered token budget, ran the registered cell at the
  registered commit, and whose final validation row carries the same token and compute figures.
* ``interpolate(points, budget)``: linear in measured compute between two bracketing points; None outside the measured
  range.
* ``envelope(points)``: Pareto-improving points only, then the lower convex hull in (log compute, loss).
* ``comparison(points)``: at nine log-spaced compute budgets, the interpolated loss of every recursion count's
  fixed-weight-decay ladder and which recursion count wins; the K = 1 ladder at fixed and at per-depth tuned weight
  decay; loop frontiers (fixed weight decay / the K = 1 tuned weight decay per depth), both cut at the largest K = 1
  compute so that frontiers are compared over the same range; the tuned weight decay of every (depth, K) whose
  weight-decay axis is complete.
(Reference: src/archlab/tracking/loop_regularization_report.py:17-167.)
"""
from __future__ import annotations

import csv
import json
import math
from collections import defaultdict
from pathlib import Path

from ..contracts.substrate import atomic_write_json
from ..train.loop_sweep import ANCHOR, RUN_TOKEN_BUDGET, WEIGHT_DECAYS, cell_name, cells, validate_cell

FIXED_WD = ANCHOR[2]


def _rows(path: Path) -> list[dict]:
    return [json.loads(line) for line in path.read_text().splitlines() if line.strip()] if path.exists() else []


def load_measurements(plan: dict) -> tuple[list[dict], list[dict]]:
    if sorted(cell_name(r["cell"]) for r in plan["runs"]) != sorted(cell_name(c) for c in cells()):
        raise ValueError("the report plan differs from the preregistered grid")
    completed, trajectories = [], []
    for run in plan["runs"]:
        cell, root = run["cell"], Path(run["output"])
        validate_cell(cell)
        rows = _rows(root / "validation.jsonl")
        for row in rows:
            if row.get("consumed_supervised_tokens", 0) > 0:
                if not math.isfinite(row["loss"]) or row["training_gpu_seconds"] <= 0:
                    raise ValueError(f"invalid validation measurement: {root}")
                trajectories.append({"cell": cell_name(cell), **cell, "loss": row["loss"], "compute": row["training_gpu_seconds"],
                                     "tokens": row["consumed_supervised_tokens"], "step": row["step"]})
        if not (root / "COMPLETE.json").exists():
            continue
        done, contract = json.loads((root / "COMPLETE.json").read_text()), json.loads((root / "RUN_CONTRACT.json").read_text())
        if (done.get("passed") is not True or done["supervised_tokens"] != RUN_TOKEN_BUDGET or contract["repeated_data_sweep"] != cell
                or contract["project_commit"] != run["source_commit"]):
            raise ValueError(f"a completed run differs from its registered contract: {root}")
        final = next((r for r in rows if r["step"] == done["step"]), None)
        if final is None or final["consumed_supervised_tokens"] != done["supervised_tokens"] or final["training_gpu_seconds"] != done["training_gpu_seconds"]:
            raise ValueError(f"a completed run lacks its final validation measurement: {root}")
        completed.append({"cell": cell_name(cell), **cell, "loss": final["loss"], "compute": final["training_gpu_seconds"], "source": str(root),
                          "source_commit": run["source_commit"]})
    return completed, trajectories


def interpolate(points: list[dict], budget: float) -> float | None:
    ordered = sorted(points, key=lambda p: p["compute"])
    for p in ordered:
        if p["compute"] == budget:
            return p["loss"]
    for a, b in zip(ordered, ordered[1:]):
        if a["compute"] < budget < b["compute"]:
            t = (budget - a["compute"]) / (b["compute"] - a["compute"])
            return a["loss"] + t * (b["loss"] - a["loss"])
    return None


def envelope(points: list[dict]) -> list[dict]:
    hull, best = [], math.inf
    for p in sorted(points, key=lambda q: (q["compute"], q["loss"])):
        if p["loss"] >= best:
            continue
        best = p["loss"]
        x = math.log(p["compute"])
        while len(hull) >= 2:
            (xa, ya), (xb, yb) = ((math.log(q["compute"]), q["loss"]) for q in hull[-2:])
            if (xb - xa) * (p["loss"] - ya) - (yb - ya) * (x - xa) > 0:       # the last point stays below the chord a -> p
                break
            hull.pop()
        hull.append(p)
    return hull


def tuned_weight_decay(points: list[dict]) -> dict[tuple[int, int], dict]:
    """Best point of every (depth, recursions) whose weight-decay axis was run completely."""
    groups = defaultdict(list)
    for p in points:
        groups[(p["reference_depth"], p["recursions"])].append(p)
    return {k: min(g, key=lambda p: p["loss"]) for k, g in groups.items() if {p["weight_decay"] for p in g} == set(WEIGHT_DECAYS)}


def comparison(points: list[dict]) -> dict:
    fixed = [p for p in points if p["weight_decay"] == FIXED_WD]
    ladders = defaultdict(list)
    for p in fixed:
        ladders[p["recursions"]].append(p)
    cuts = []
    if points:
        low, high = min(p["compute"] for p in points), max(p["compute"] for p in points)
        for i in range(9):
            budget = math.exp(math.log(low) + i / 8 * math.log(high / low))
            losses = {k: v for k, v in ((k, interpolate(g, budget)) for k, g in sorted(ladders.items())) if v is not None}
            if len(losses) >= 2:
                cuts.append({"compute": budget, "losses": losses, "best_k": min(losses, key=losses.get)})
    tuned = tuned_weight_decay(points)
    k1_tuned = [p for (d, k), p in sorted(tuned.items()) if k == 1]
    tuned_pool = [p for best in k1_tuned for p in points if p["reference_depth"] == best["reference_depth"] and p["weight_decay"] == best["weight_decay"]]
    k1_fixed = sorted((p for p in fixed if p["recursions"] == 1), key=lambda p: p["compute"])
    eligible = [p for p in fixed if (p["reference_depth"], p["recursions"]) != (4, 6)]        # the recipe convention: d4 exists only at K = 6
    frontiers = [envelope(eligible), envelope(tuned_pool)]
    if k1_fixed:
        cap = k1_fixed[-1]["compute"]
        frontiers = [f[:next((j + 1 for j, p in enumerate(f) if p["compute"] >= cap), len(f))] for f in frontiers]
    return {"cuts": cuts,
            "recipes": {"K1, fixed weight decay": k1_fixed, "K1, tuned weight decay": sorted(k1_tuned, key=lambda p: p["compute"]),
                        "loop frontier, fixed weight decay": frontiers[0], "loop frontier, K1-tuned weight decay": frontiers[1]},
            "optimal_weight_decay": [{"reference_depth": d, "recursions": k, "weight_decay": p["weight_decay"]} for (d, k), p in sorted(tuned.items())]}


def report(plan_path, output) -> dict:
    plan, output = json.loads(Path(plan_path).read_text()), Path(output)
    output.mkdir(parents=True, exist_ok=True)
    completed, trajectories = load_measurements(plan)
    analysis = comparison(completed)
    fields = ["cell", "reference_depth", "stored_layers", "hidden_size", "recursions", "weight_decay", "loss", "compute"]
    for name, rows, extra in (("final.csv", completed, ["source_commit"]), ("trajectories.csv", trajectories, ["tokens", "step"])):
        with (output / name).open("w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=fields + extra, extrasaction="ignore")
            w.writeheader()
            w.writerows(rows)
    summary = {"format": "archlab-loop-sweep-report-v1", "registered_cells": len(plan["runs"]), "completed_cells": len(completed),
               "trajectory_points": len(trajectories), "cells_sha256": plan.get("cells_sha256"), "analysis": analysis,
               "note": "final-loss comparisons use exact-budget completed cells only; no extrapolation beyond measured compute"}
    atomic_write_json(output / "report.json", summary)
    return summary
