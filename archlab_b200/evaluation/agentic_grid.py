"""A fixed (task x seed) evaluation grid for agentic policies: auditable, resumable, and honest about what is missing.

* ``sample_seed(task, seed)``: one deterministic random stream per grid cell, shared by every checkpoint evaluated on
  the grid (differences between checkpoints are then paired by construction).
* ``completed_records``: rows outside the declared grid, duplicate scored cells and non-binary rewards are errors.
* ``summarize``: pass@1 and its task-bootstrap interval exist ONLY for a complete grid; until then the summary reports
  how many cells are scored or missing and a clearly named provisional mean over the tasks whose seeds are all in.  A
  cell that failed for infrastructure reasons stays missing -- it never becomes a zero and never leaves the denominator.
* ``bind_invocation``: an output directory belongs to one evaluation contract.  Re-running may only EXTEND the seed list
  (a prefix-preserving expansion); anything else needs a new directory.  The superseded invocation is kept beside it.
* ``paired_difference``: two complete grids over the same tasks and seeds, task-level differences, paired bootstrap.
* ``error_outcome`` / ``policy_cap_reason``: what a failed or capped episode may be called.  A wall-clock timeout that
  also covers resource waits is not a model failure; a backend failure that is not a context overflow is ungradable.
(Reference: src/archlab/evaluation/agentic_curve.py:32-143.)
"""
from __future__ import annotations

import hashlib
import json
from collections import Counter
from pathlib import Path

import numpy as np

from ..contracts.substrate import atomic_write_json, sha256_file

SCHEMA = "archlab-agentic-evaluation-v1"
DEFAULT_SEEDS = (101, 211, 307, 401, 503, 601, 701, 809)
FULL_GRID = (48, 8)                                  # tasks, seeds below which a result is labelled preliminary
CONTEXT_MARKERS = ("maximum context length", "max_model_len", "trajectory capacity", "context length exceeded")
_BOOTSTRAP_SEED = 20261017


def sample_seed(task: str, seed: int) -> int:
    return int(hashlib.sha256(f"{task}\0{seed}".encode()).hexdigest()[:8], 16)


def completed_records(records: list[dict], tasks: list[str], seeds: list[int]):
    expected = {(t, s) for t in tasks for s in seeds}
    done = {}
    for row in records:
        key = (row["task"], row["seed"])
        if key not in expected:
            raise ValueError(f"episode outside the declared grid: {key}")
        if row.get("status") != "scored":
            continue
        if key in done:
            raise ValueError(f"duplicate scored episode: {key}")
        if row.get("reward") not in (0.0, 1.0):
            raise ValueError(f"expected a binary executable reward: {key}")
        done[key] = row
    return expected, done


def summarize(records: list[dict], tasks: list[str], seeds: list[int], *, bootstrap: int = 2000) -> dict:
    expected, done = completed_records(records, tasks, seeds)
    per_task = {t: [done[(t, s)]["reward"] for s in seeds if (t, s) in done] for t in tasks}
    full = {t: sum(v) / len(seeds) for t, v in per_task.items() if len(v) == len(seeds)}
    complete = len(done) == len(expected)
    total = lambda key: sum(r.get(key, 0) for r in done.values())
    out = {"schema": SCHEMA, "complete": complete, "preliminary": len(tasks) < FULL_GRID[0] or len(seeds) < FULL_GRID[1],
           "expected_samples": len(expected), "scored_samples": len(done), "missing_samples": len(expected) - len(done), "task_count": len(tasks),
           "complete_task_count": len(full), "samples_per_task": len(seeds), "pass_at_1": None, "success_at_k": None, "task_bootstrap_95ci": None,
           "provisional_complete_task_pass_at_1": sum(full.values()) / len(full) if full else None,
           "per_task": {t: {"scored": len(v), "successes": sum(v), "expected": len(seeds)} for t, v in per_task.items()},
           "infrastructure_attempts": sum(r.get("status") == "missing" for r in records),
           "terminations": dict(Counter(r.get("termination", "unknown") for r in done.values())),
           "cap_reasons": dict(Counter(r.get("cap_reason", "none") for r in done.values())),
           "length_limited_calls": total("length_limited_calls"), "generation_calls": total("generation_calls"),
           "generated_tokens": total("generated_tokens"), "episode_seconds": total("seconds")}
    if complete:
        values = np.asarray(list(full.values()), dtype=float)
        draws = np.random.default_rng(_BOOTSTRAP_SEED).choice(values, size=(bootstrap, len(values)), replace=True).mean(axis=1)
        out.update(pass_at_1=float(values.mean()), success_at_k=sum(any(v) for v in per_task.values()) / len(tasks),
                   task_bootstrap_95ci=[float(x) for x in np.quantile(draws, [0.025, 0.975])])
    return out


def bind_invocation(path, invocation: dict) -> None:
    path = Path(path)
    new = json.loads(json.dumps(invocation))
    if path.exists():
        old = json.loads(path.read_text())
        fixed = lambda d: {k: v for k, v in d.items() if k not in ("seeds", "scope")}
        old_seeds, new_seeds = old.get("seeds", []), new.get("seeds", [])
        if fixed(old) != fixed(new) or new_seeds[:len(old_seeds)] != old_seeds:
            raise ValueError("the output holds a different evaluation contract; use a new directory")
        if old != new:
            atomic_write_json(path.with_name(f"invocation-{sha256_file(path)}.json"), old)
    atomic_write_json(path, new)


def paired_difference(left: list[dict], right: list[dict], tasks: list[str], seeds: list[int], *, bootstrap: int = 2000) -> dict:
    expected, a = completed_records(left, tasks, seeds)
    _, b = completed_records(right, tasks, seeds)
    if set(a) != expected or set(b) != expected:
        raise ValueError("a paired comparison requires both grids to be complete")
    values = np.asarray([sum(b[(t, s)]["reward"] - a[(t, s)]["reward"] for s in seeds) / len(seeds) for t in tasks])
    draws = np.random.default_rng(_BOOTSTRAP_SEED).choice(values, size=(bootstrap, len(values)), replace=True).mean(axis=1)
    return {"delta_pass_at_1": float(values.mean()), "task_paired_95ci": [float(x) for x in np.quantile(draws, [0.025, 0.975])]}


def error_outcome(error: BaseException) -> dict:
    wall = isinstance(error, TimeoutError) and "wall timeout" in str(error)
    return {"status": "missing", "reward": None, "termination": "wall_budget_unclassified" if wall else "infrastructure_or_unclassified",
            "error_type": type(error).__name__}


def policy_cap_reason(reward_info: dict, turns: int, *, turn_limit: int = 300) -> str:
    detail = str(reward_info.get("result", "")).lower()
    context = any(m in detail for m in CONTEXT_MARKERS)
    if str(reward_info.get("agent_status")) == "ModelQueryError" and not context:
        raise RuntimeError("ungradable model backend failure")
    if reward_info.get("agent_completed"):
        return "none"
    if turns >= turn_limit:
        return "turn_limit"
    return "context_limit" if context else "unfinished_other"
