"""Offline evaluation and rollout analysis that stays out of the training hot path.

* checkpoint ladder: which exported checkpoints still need scoring under a JSON plan (fixed points, the
  newest export once it is ``every`` steps past the last scored one, every export at a multiple of
  ``every``), with an idempotent ledger so that a point is logged once
  (src/archlab/evaluation/ladder.py:24-60);
* paired capability statistics between a base and an adapted model on the SAME cases: accuracy
  difference with a normal-approximation interval over the paired differences, discordant counts and the
  exact two-sided sign (McNemar) test (src/archlab/evaluation/capability.py:106-186);
* modular pair-search probes with exact answers: a NO instance and a YES twin that differ in one entry
  (src/archlab/evaluation/pair_search.py:20-80);
* trajectory replay windows: keep at most half a window of prompt, score only generated tokens
  (src/archlab/evaluation/trajectory_replay.py:19-60);
* agentic rollout accounting from session logs: wasted groups (every rollout failed - no GRPO gradient),
  per-task learning within a data period, and the rows worth sampling next
  (src/archlab/rl/rollouts.py:24-100).
"""
from __future__ import annotations

import json
import math
import random
from collections import defaultdict
from pathlib import Path
from statistics import NormalDist

import numpy as np


# ------------------------------------------------------------------------------------------------
# ladder
# ------------------------------------------------------------------------------------------------
def exported_steps(exports: Path, prefix: str) -> list[int]:
    steps = []
    for path in Path(exports).glob(f"{prefix}-step*"):
        tail = path.name[len(prefix) + 5:]
        if tail.isdigit() and (path / "EXPORTED").exists():
            steps.append(int(tail))
    return sorted(steps)


def ladder_candidates(plan: dict, done: set[str]) -> list[dict]:
    found, seen = [], set(done)
    for entry in plan["points"]:
        if "newest" in entry:
            spec = entry["newest"]
            steps = exported_steps(spec["exports"], spec["prefix"])
            ran = [s for s in steps if f"{spec['prefix']}-step{s}" in done]
            points = [(steps[-1], spec)] if steps and (not ran or steps[-1] - max(ran) >= spec["every"]) else []
        elif "every" in entry:
            spec = entry["every"]
            points = [(s, spec) for s in exported_steps(spec["exports"], spec["prefix"]) if s % spec["every"] == 0]
        else:
            if Path(entry["model"]).exists():
                found.append(entry)
            continue
        for step, spec in points:
            label = f"{spec['prefix']}-step{step}"
            if label not in seen:
                seen.add(label)
                found.append({"label": label, "model": str(Path(spec["exports"]) / label), "curve": spec["curve"], "step": step})
    return [p for p in found if p["label"] not in done]


class PointLedger:
    """Append-only record of scored points; ``record`` is a no-op for a label that is already there."""

    def __init__(self, path: Path):
        self.path = Path(path)

    def done(self) -> set[str]:
        if not self.path.exists():
            return set()
        return {json.loads(l)["label"] for l in self.path.read_text().splitlines() if l}

    def record(self, label: str, **fields) -> bool:
        if label in self.done():
            return False
        self.path.parent.mkdir(parents=True, exist_ok=True)
        with open(self.path, "a") as f:
            f.write(json.dumps({"label": label, **fields}, sort_keys=True) + "\n")
        return True


# ------------------------------------------------------------------------------------------------
# paired statistics
# ------------------------------------------------------------------------------------------------
def paired_statistics(base: list[int], adapted: list[int], confidence: float = 0.95) -> dict:
    if len(base) != len(adapted) or not base:
        raise ValueError("paired evaluation needs the same non-empty case list")
    if any(v not in (0, 1) for v in (*base, *adapted)):
        raise ValueError("outcomes are 0 or 1")
    n = len(base)
    diffs = [a - b for a, b in zip(adapted, base)]
    mean = sum(diffs) / n
    var = sum((d - mean) ** 2 for d in diffs) / (n - 1) if n > 1 else 0.0
    half = NormalDist().inv_cdf(0.5 + confidence / 2) * math.sqrt(var / n)
    gained, lost = sum(d == 1 for d in diffs), sum(d == -1 for d in diffs)
    m = gained + lost
    tail = sum(math.comb(m, k) for k in range(0, min(gained, lost) + 1)) / 2 ** m if m else 0.5
    return {"cases": n, "base_accuracy": sum(base) / n, "adapted_accuracy": sum(adapted) / n, "difference": mean,
            "interval": [mean - half, mean + half], "gained": gained, "lost": lost, "sign_test_p": min(1.0, 2 * tail)}


def select_cases(rows: list[dict], *, limits: dict[str, int], seed: int) -> list[dict]:
    """Deterministic per-suite subsample: shuffle each suite with its own seeded stream, keep ``limits[suite]``."""
    out = []
    for suite in sorted(limits):
        pool = sorted((r for r in rows if r["suite"] == suite), key=lambda r: str(r["id"]))
        random.Random(f"{seed}:{suite}").shuffle(pool)
        if len(pool) < limits[suite]:
            raise ValueError(f"suite {suite} has only {len(pool)} cases")
        out += pool[: limits[suite]]
    return out


# ------------------------------------------------------------------------------------------------
# pair-search probes
# ------------------------------------------------------------------------------------------------
def witnesses(recent, earlier, target, modulus):
    """All (i, j) with recent[i] + earlier[j] == target (mod modulus), component-wise."""
    where = {tuple(v): j for j, v in enumerate(earlier)}
    out = []
    for i, (x, y) in enumerate(recent):
        c = ((target[0] - x) % modulus, (target[1] - y) % modulus)
        if c in where:
            out.append((i, where[c]))
    return out


def make_twins(rng: random.Random, *, earlier_count: int, recent_count: int = 2, modulus: int = 97) -> dict:
    """A NO instance (no witness) and a YES twin with exactly one witness; the twins differ in one earlier entry."""
    while True:
        pair = lambda: (rng.randrange(modulus), rng.randrange(modulus))
        earlier = []
        while len(earlier) < earlier_count:
            p = pair()
            if p not in earlier:
                earlier.append(p)
        recent = [pair() for _ in range(recent_count)]
        target = pair()
        if witnesses(recent, earlier, target, modulus):
            continue
        i, j = rng.randrange(recent_count), rng.randrange(earlier_count)
        planted = ((target[0] - recent[i][0]) % modulus, (target[1] - recent[i][1]) % modulus)
        yes = list(earlier)
        if planted in yes:
            continue
        yes[j] = planted
        if witnesses(recent, yes, target, modulus) == [(i, j)]:
            return {"target": target, "recent": recent, "no": earlier, "yes": yes, "witness": (i, j), "modulus": modulus}


# ------------------------------------------------------------------------------------------------
# trajectory replay
# ------------------------------------------------------------------------------------------------
def replay_window(prompt: np.ndarray, response: np.ndarray, generated: np.ndarray, length: int):
    """-> (tokens [<= length], score mask aligned with next-token targets, generated tokens scored).

    Up to half the window goes to the END of the prompt; the rest is filled from the start of the
    response; only positions whose target is a generated (not tool-inserted) token are scored."""
    if length < 2:
        raise ValueError("a window needs at least two tokens")
    if response.shape != generated.shape:
        raise ValueError("generated mask must align with the response")
    keep_prompt = min(len(prompt), length // 2)
    keep_resp = min(len(response), length - keep_prompt)
    tokens = np.concatenate([prompt[len(prompt) - keep_prompt:], response[:keep_resp]])
    mask = np.zeros(len(tokens) - 1, dtype=bool)
    mask[keep_prompt - 1:] = generated[:keep_resp].astype(bool)[: len(mask) - (keep_prompt - 1)] if keep_prompt else \
        generated[1:keep_resp].astype(bool)
    return tokens, mask, int(mask.sum())


# ------------------------------------------------------------------------------------------------
# rollout accounting
# ------------------------------------------------------------------------------------------------
def read_sessions(agents: Path, first: int = 0, last: int = 10 ** 9) -> list[dict]:
    rows = []
    for step_dir in Path(agents).glob("step_*"):
        step = int(step_dir.name.split("_")[1])
        if not first <= step <= last:
            continue
        for path in step_dir.glob("session-*/session.json"):
            try:
                info = json.loads(path.read_text())
            except (OSError, ValueError):
                continue
            rows.append({"step": step, "task": info["dataset_index"], "win": (info.get("reward_score") or 0) > 0,
                         "turns": info.get("num_turns") or 0})
    return rows


def bootstrap_mean(values: list[float], *, draws: int = 2000, seed: int = 0):
    rng = random.Random(seed)
    n = len(values)
    means = sorted(sum(rng.choice(values) for _ in range(n)) / n for _ in range(draws))
    return sum(values) / n, [means[int(0.025 * draws)], means[int(0.975 * draws) - 1]]


def waste(rows: list[dict]) -> dict:
    groups = defaultdict(list)
    for r in rows:
        groups[(r["step"], r["task"])].append(r["win"])
    dead = [g for g in groups.values() if not any(g)]
    solved = [g for g in groups.values() if all(g)]
    return {"groups": len(groups), "all_failed": len(dead), "all_failed_share": len(dead) / max(1, len(groups)),
            "all_solved": len(solved), "informative": len(groups) - len(dead) - len(solved)}


def learning(rows: list[dict]) -> dict:
    """Per task: success rate on later visits minus the first visit (tasks seen at two or more steps)."""
    by_task = defaultdict(lambda: defaultdict(list))
    for r in rows:
        by_task[r["task"]][r["step"]].append(r["win"])
    gains = []
    for visits in by_task.values():
        steps = sorted(visits)
        if len(steps) < 2:
            continue
        first = sum(visits[steps[0]]) / len(visits[steps[0]])
        later = [w for s in steps[1:] for w in visits[s]]
        gains.append(sum(later) / len(later) - first)
    if not gains:
        return {"tasks": 0, "gain": None, "interval": None}
    mean, ci = bootstrap_mean(gains)
    return {"tasks": len(gains), "gain": mean, "interval": ci}


def learnable_rows(rows: list[dict], total: int, label: str, recheck: float = 0.15) -> list[int]:
    """Rows to sample next: solved on the last visit, never visited, or a deterministic (hash-seeded) re-check of
    ``recheck`` of the tasks that failed last time."""
    last = {}
    for r in sorted(rows, key=lambda r: r["step"]):
        last.setdefault(r["task"], {})[r["step"]] = last.get(r["task"], {}).get(r["step"], False) or r["win"]
    keep = []
    for task in range(total):
        if task not in last:
            keep.append(task)
            continue
        final = last[task][max(last[task])]
        if final or random.Random(f"{label}:{task}").random() < recheck:
            keep.append(task)
    return keep
