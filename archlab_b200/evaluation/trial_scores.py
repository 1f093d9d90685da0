"""Scoring a finished job of an external agent-benchmark harness (one ``result.json`` per trial under the job directory).

* ``complete_job(jobs, label)``: the newest-sorted run of ``label`` whose harness statistics show no running and no
  pending trial -- a job that is still moving is never scored.
* ``score_trials(job)``: mean reward over ALL trials, with an errored trial counting as 0 (the leaderboard's rule, so a
  crash cannot raise the score by shrinking the denominator), a bootstrap 95 % interval over trials, the solved tasks,
  and the errors by type.  ``valid`` (tasks whose reference solution passes at this site) adds the same mean over that
  subset, which separates limits of the local environment from limits of the model.
(Reference: src/archlab/evaluation/tb21.py:61-94.)
"""
from __future__ import annotations

import json
import random
from collections import Counter
from pathlib import Path


def complete_job(jobs, label: str) -> Path | None:
    for result in sorted((Path(jobs) / label).glob("*/result.json")):
        stats = json.loads(result.read_text()).get("stats", {})
        if stats.get("n_running_trials") == 0 and stats.get("n_pending_trials") == 0:
            return result.parent
    return None


def read_trials(job) -> list[dict]:
    rows = []
    for path in sorted(Path(job).glob("*/result.json")):
        record = json.loads(path.read_text())
        reward = ((record.get("verifier_result") or {}).get("rewards") or {}).get("reward")
        rows.append({"task": record.get("task_name"), "reward": float(reward or 0.0), "error": (record.get("exception_info") or {}).get("exception_type")})
    if not rows:
        raise ValueError(f"no trials in {job}")
    return rows


def score_trials(job, *, bootstrap: int = 2000, valid: set[str] | None = None, seed: int = 0) -> dict:
    rows = read_trials(job)
    rewards = [r["reward"] for r in rows]
    n, rng = len(rewards), random.Random(seed)
    means = sorted(sum(rng.choice(rewards) for _ in range(n)) / n for _ in range(bootstrap))
    out = {"mean_reward": sum(rewards) / n, "ci95": [means[int(0.025 * bootstrap)], means[int(0.975 * bootstrap) - 1]], "trials": n,
           "solved": sum(r >= 1.0 for r in rewards), "solved_tasks": sorted(r["task"] for r in rows if r["reward"] >= 1.0),
           "errors": dict(Counter(r["error"] for r in rows if r["error"]))}
    if valid:
        inside = [r["reward"] for r in rows if r["task"] in valid]
        out["oracle_valid"] = {"tasks": len(inside), "mean_reward": sum(inside) / max(1, len(inside))}
    return out
