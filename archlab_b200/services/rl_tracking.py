"""RL runs in the tracking store: a whitelist of metrics with their ranges, and a sidecar that tails the learner's
ledgers exactly once.

Only metrics named in the tables below are published; each carries a constraint (a rate in [0, 1], a non-negative
measurement, a non-negative integer count) and a non-finite or out-of-range value stops the sync instead of being
plotted.  A missing KL is not published as zero (``reference_kl_available: false`` suppresses it); rollout throughput
is derived from tokens / seconds only when seconds is positive; two aliases of one metric must agree.

``RLMetricSync`` keeps a byte cursor per ledger file in its state (one writer at a time), reads only complete lines,
requires the update step to be non-decreasing within a ledger, and publishes ``(metric, value, step, time)`` points
through the same store interface as the training sidecar.  (Reference: src/archlab/tracking/rl_mlflow.py:40-163,233-537.)
"""
from __future__ import annotations

import json
import math
import time
from pathlib import Path

from ..contracts.substrate import atomic_write_json
from .tracking import SingleWriterLock

RATE, MEASURE, COUNT, FREE = "rate", "measure", "count", "free"

TRAIN = {   # ledger key -> (published name, constraint)
    "reward_mean": ("rl/reward_mean", FREE), "reward_std": ("rl/reward_std", MEASURE), "policy_loss": ("rl/policy_loss", FREE),
    "valid_answer_rate": ("rl/valid_answer_rate", RATE), "truncation_rate": ("rl/truncation_rate", RATE),
    "nonflat_prompt_groups": ("rl/nonflat_prompt_groups", COUNT), "optimizer_step": ("rl/optimizer_step", COUNT),
    "update_skipped": ("rl/update_skipped", RATE), "skip_update": ("rl/update_skipped", RATE),
    "replay_max_abs_error": ("numerical/replay_max_abs_error", MEASURE), "replay_mean_abs_error": ("numerical/replay_mean_abs_error", MEASURE),
    "rollout_tokens_per_second": ("perf/rollout_tokens_per_second", MEASURE), "generated_tokens_per_second": ("perf/generated_tokens_per_second", MEASURE),
    "iteration_seconds": ("perf/iteration_seconds", MEASURE), "update_seconds": ("perf/update_seconds", MEASURE),
    "rollout_seconds": ("perf/rollout_seconds", MEASURE), "gradient_norm": ("optim/gradient_norm", MEASURE),
    "learning_rate": ("optim/learning_rate", MEASURE),
}
EVAL = {"pass_at_1": RATE, "valid_answer_rate": RATE, "truncation_rate": RATE, "examples": MEASURE, "seconds": MEASURE}
PROFILE_FORMAT = "archlab-rl-rollout-throughput-v1"


def _number(value, name: str, constraint: str = FREE) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        if isinstance(value, bool):
            value = float(value)
        else:
            raise ValueError(f"invalid scalar for {name}")
    v = float(value)
    if constraint == RATE and not 0 <= v <= 1:
        raise ValueError(f"{name} must lie in [0, 1]")
    if constraint in (MEASURE, COUNT) and v < 0:
        raise ValueError(f"{name} must be non-negative")
    if constraint == COUNT and not v.is_integer():
        raise ValueError(f"{name} must be an integer")
    return v


def update_step(row: dict) -> int:
    value = row.get("update_step", row.get("step", row.get("policy_version")))
    if type(value) is not int or value < 0:
        raise ValueError("a metric record needs a non-negative integer update_step")
    return value


def train_values(row: dict) -> dict[str, float]:
    out: dict[str, float] = {}
    for key, (name, constraint) in TRAIN.items():
        value = row.get(key, row.get(name))
        if value is None:
            continue
        v = _number(value, name, constraint)
        if out.setdefault(name, v) != v:
            raise ValueError(f"conflicting aliases for {name}")
    if row.get("reference_kl_available", True):
        kl = row.get("sampled_kl", row.get("kl", row.get("rl/kl")))
        if kl is not None:
            out["rl/kl"] = _number(kl, "rl/kl")
    if type(row.get("policy_version")) is int:
        out["rl/policy_version"] = float(row["policy_version"])
    if "perf/rollout_tokens_per_second" not in out and "rollout_tokens" in row:
        seconds = out.get("perf/rollout_seconds", 0.0)
        if seconds <= 0:
            raise ValueError("rollout throughput requires a positive rollout_seconds")
        out["perf/rollout_tokens_per_second"] = _number(row["rollout_tokens"], "rollout_tokens", MEASURE) / seconds
    if not out:
        raise ValueError("the record has no recognised RL metrics")
    return out


def evaluation_values(row: dict) -> dict[str, float]:
    out = {}
    for key, constraint in EVAL.items():
        value = row.get(key, row.get("eval/" + key))
        if value is not None:
            out["eval/" + key] = _number(value, "eval/" + key, constraint)
    if "eval/pass_at_1" not in out:
        raise ValueError("an evaluation record needs pass_at_1")
    if type(row.get("policy_version")) is int:
        out["eval/policy_version"] = float(row["policy_version"])
    return out


def profile_values(profile: dict) -> dict[str, float]:
    """Measured scalars of a rollout-throughput profile; never inputs, paths or derived utilisation."""
    if profile.get("format") != PROFILE_FORMAT:
        raise ValueError("unrecognised rollout profile format")
    out = {f"profile/{k}": _number(profile[k], k, MEASURE) for k in ("batch4_over_batch1_throughput_ratio", "prompt_tokens", "max_new_tokens", "world_size",
                                                                      "retained_weights") if profile.get(k) is not None}
    sizes = set()
    for batch in profile.get("batches", []):
        size = batch.get("batch_size_per_rank")
        if type(size) is not int or not 1 <= size <= 1024 or size in sizes:
            raise ValueError("profile batch sizes must be distinct integers in 1..1024")
        sizes.add(size)
        for k in ("generated_tokens_per_second", "max_rank_seconds_sum", "actual_generated_tokens_global", "input_tokens_processed_global", "global_batch_size"):
            if batch.get(k) is not None:
                out[f"profile/batch_{size}/{k}"] = _number(batch[k], k, MEASURE)
    if not out:
        raise ValueError("the profile holds no measured scalars")
    return out


class RLMetricSync:
    LEDGERS = {"train": ("metrics.jsonl", train_values), "evaluation": ("evaluation.jsonl", evaluation_values)}

    def __init__(self, store, state_path, *, clock=time.time):
        self.store, self.state_path, self.clock = store, Path(state_path), clock
        self.state = {"runs": {}}

    def _tail(self, path: Path, cursor: dict) -> list[dict]:
        """Complete lines after the cursor; the cursor moves only past lines that were returned."""
        if not path.exists():
            return []
        size = path.stat().st_size
        if size < cursor["offset"]:
            raise ValueError(f"{path.name} shrank; ledgers are append-only")
        with path.open("rb") as f:
            f.seek(cursor["offset"])
            data = f.read()
        end = data.rfind(b"\n") + 1
        rows = [json.loads(line) for line in data[:end].splitlines() if line.strip()]
        cursor["offset"] += end
        return rows

    def sync_run(self, spec: dict) -> dict:
        """``spec``: ``{"source_id", "name", "root", "tags"}``."""
        root = Path(spec["root"])
        with SingleWriterLock(self.state_path.with_suffix(".lock")):
            if self.state_path.exists():                              # another sidecar instance may have advanced the cursors
                self.state = json.loads(self.state_path.read_text())
            run = self.state["runs"].setdefault(spec["source_id"], {"run_id": None, "cursors": {}, "last_step": {}})
            if run["run_id"] is None:
                found = self.store.find_runs(spec["source_id"])
                if len(found) > 1:
                    raise ValueError(f"several tracked runs claim {spec['source_id']}")
                run["run_id"] = found[0] if found else self.store.create_run(spec["source_id"], spec["name"], spec.get("tags", {}))
            sent = {}
            for kind, (filename, convert) in self.LEDGERS.items():
                cursor = run["cursors"].setdefault(kind, {"offset": 0})
                before = dict(cursor)
                try:
                    rows = self._tail(root / filename, cursor)
                    points, last = [], run["last_step"].get(kind, -1)
                    for row in rows:
                        step = update_step(row)
                        if step < last:
                            raise ValueError(f"{filename}: update step went backwards ({step} after {last})")
                        last = step
                        stamp = int(1000 * row.get("time", self.clock()))
                        points += [(name, value, step, stamp) for name, value in convert(row).items()]
                    self.store.log_points(run["run_id"], points)
                except Exception:
                    run["cursors"][kind] = before                     # nothing of this ledger counts as sent
                    atomic_write_json(self.state_path, self.state)
                    raise
                run["last_step"][kind] = last
                sent[kind] = len(rows)
            profile = root / "rollout_profile.json"
            if profile.exists() and not run.get("profile_sent"):
                values = profile_values(json.loads(profile.read_text()))
                self.store.set_fields(run["run_id"], params={k: v for k, v in values.items()})
                run["profile_sent"] = True
            atomic_write_json(self.state_path, self.state)
        return {"run_id": run["run_id"], "rows": sent}
