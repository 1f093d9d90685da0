"""Keep one training arm running to its step budget without a person in the loop.

An arm spec names the base config, the checkpoint directory, the current data snapshot and the source
snapshot.  ``tick()`` is one pass of the loop (the entry point runs it every two minutes):

* trainer alive, launch inputs unchanged  -> nothing to do;
* trainer alive, data / source / base config changed -> ask it to stop right after its NEXT saved
  checkpoint (never mid-interval: the latest-iteration marker is the last file a save writes);
* trainer gone, budget reached -> done;
* trainer gone otherwise -> wait until the GPUs are free, then resume from the newest complete
  checkpoint.  A new data snapshot resumes model state only with a fresh loader (seed 1000 + step);
  anything else resumes the full checkpoint with the recorded seed.

Every launch is appended to ``LAUNCHES.jsonl``.  Three launches in a row that produce no new checkpoint
end the supervision with an error.  Process control (is the trainer alive, are GPUs free, start, stop)
is behind a small ``Ops`` interface so that the policy is testable without a cluster.  Follows the
policy of the reference's supervisor (src/archlab/training/supervise.py:99-247).
"""
from __future__ import annotations

import hashlib
import json
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Protocol


def rotate_log(path: Path) -> Path | None:
    """Move a non-empty log aside under a time-stamped name; never overwrites an earlier rotation."""
    path = Path(path)
    if not (path.exists() and path.stat().st_size):
        return None
    stem = f"{path.stem}-{time.strftime('%m%d-%H%M%S')}"
    target, n = path.with_name(stem + path.suffix), 1
    while target.exists():
        n += 1
        target = path.with_name(f"{stem}-{n}{path.suffix}")
    path.rename(target)
    return target


def base_digest(spec: dict) -> str:
    return hashlib.sha256(Path(spec["base"]).read_bytes()).hexdigest()[:16]


def last_launch(path: Path) -> dict:
    lines = Path(path).read_text().splitlines() if Path(path).exists() else []
    return json.loads(lines[-1]) if lines else {}


def plan_launch(spec: dict, step: int, last: dict) -> dict:
    fresh = spec["data"] != last.get("data") or (step == last.get("step") and last.get("mode") == "fresh")
    return {"step": step, "data": spec["data"], "source": spec["source"], "base": base_digest(spec),
            "mode": "fresh" if fresh else "full", "seed": 1000 + step if fresh else last.get("seed", 1000 + step)}


def switch_due(spec: dict, last: dict) -> bool:
    return bool(last) and (spec["data"] != last.get("data") or spec["source"] != last.get("source")
                           or last.get("base", base_digest(spec)) != base_digest(spec))


def latest_checkpoint_step(ckpt_dir: Path, marker: str = "latest_checkpointed_iteration.txt") -> int:
    """Step of the newest COMPLETE checkpoint (the marker file is written last), 0 when none."""
    p = Path(ckpt_dir) / marker
    try:
        return int(p.read_text().strip())
    except (FileNotFoundError, ValueError):
        return 0


class Ops(Protocol):
    def trainer_alive(self) -> bool: ...
    def gpus_free(self) -> bool: ...
    def start(self, launch: dict, resume_from: str | None) -> None: ...
    def request_stop_after_checkpoint(self) -> None: ...


@dataclass
class Verdict:
    action: str            # idle | switch_requested | waiting_for_gpus | launched | done | gave_up
    detail: dict


class Supervisor:
    def __init__(self, spec: dict, ops: Ops, *, max_stalled_launches: int = 3):
        for key in ("arm", "base", "dir", "checkpoints", "data", "source", "total_steps"):
            if key not in spec:
                raise ValueError(f"arm spec is missing {key!r}")
        self.spec, self.ops, self.max_stalled = spec, ops, max_stalled_launches
        self.dir = Path(spec["dir"])
        self.launches = self.dir / "LAUNCHES.jsonl"
        self._switch_sent_for: dict | None = None

    def _stalled(self) -> int:
        """Trailing launches recorded at the same step (no checkpoint between them)."""
        if not self.launches.exists():
            return 0
        steps = [json.loads(l)["step"] for l in self.launches.read_text().splitlines() if l]
        n = 0
        for s in reversed(steps):
            if s != steps[-1]:
                break
            n += 1
        return n

    def tick(self) -> Verdict:
        spec, last = self.spec, last_launch(self.launches)
        step = latest_checkpoint_step(spec["checkpoints"])
        if self.ops.trainer_alive():
            if switch_due(spec, last):
                key = {"data": spec["data"], "source": spec["source"], "base": base_digest(spec)}
                if self._switch_sent_for != key:
                    self.ops.request_stop_after_checkpoint()
                    self._switch_sent_for = key
                return Verdict("switch_requested", key)
            return Verdict("idle", {"step": step})
        if step >= int(spec["total_steps"]):
            return Verdict("done", {"step": step})
        if last and step == last.get("step") and self._stalled() >= self.max_stalled:
            return Verdict("gave_up", {"step": step, "launches_without_checkpoint": self._stalled()})
        if not self.ops.gpus_free():
            return Verdict("waiting_for_gpus", {"step": step})
        launch = plan_launch(spec, step, last)
        resume = None if step == 0 else str(Path(spec["checkpoints"]) / f"global_step_{step}")
        self.dir.mkdir(parents=True, exist_ok=True)
        with open(self.launches, "a") as f:
            f.write(json.dumps({**launch, "time": time.strftime("%F %T")}, sort_keys=True) + "\n")
        self.ops.start(launch, resume)
        self._switch_sent_for = None
        return Verdict("launched", {**launch, "resume_from": resume})

    def run(self, *, period_seconds: float = 120.0, sleep=time.sleep, max_ticks: int | None = None) -> Verdict:
        n = 0
        while True:
            v = self.tick()
            n += 1
            if v.action in ("done", "gave_up") or (max_ticks is not None and n >= max_ticks):
                return v
            sleep(period_seconds)
