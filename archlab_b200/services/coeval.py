"""Running evaluation on the same node as a training job without ever getting in its way.

``CoEvaluator`` runs a list of evaluation phases (commands) one after another as child processes in their OWN session and
polls a guard while each runs.  The guard yields the node back -- stops the child, records why, and ends the queue --
when GPU or host memory headroom falls under its floor, when the trainer's metrics ledger goes stale, when a trainer
announces completion (the training queue is about to advance), or when a STOP file appears.  It signals only the process
group of the child it started itself, never a trainer's; probes for free memory are injected, so the supervisor itself
needs no GPU.  A measured slowdown of the trainer against the baseline taken before the first phase is reported with
every phase receipt.  (Reference: src/archlab/evaluation/concurrent_reasoning.py:18-200.)
"""
from __future__ import annotations

import json
import os
import signal
import statistics
import subprocess
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from ..contracts.substrate import atomic_write_json


def tail_metrics(path, count: int = 64, *, window_bytes: int = 512 << 10) -> dict:
    """Median update time and throughput of the last ``count`` complete rows of a trainer's ledger (only the tail of the
    file is read; half-written or foreign lines are skipped)."""
    path = Path(path)
    with path.open("rb") as f:
        f.seek(0, 2)
        size = f.tell()
        f.seek(max(0, size - window_bytes))
        lines = f.read().splitlines()
    rows = []
    for line in lines:
        try:
            row = json.loads(line)
        except (ValueError, UnicodeError):
            continue
        if isinstance(row, dict) and "seconds" in row and "step" in row:
            rows.append(row)
    if not rows:
        raise ValueError("the training run has no completed metrics")
    rows = rows[-count:]
    return {"step": rows[-1]["step"], "median_seconds": statistics.median(r["seconds"] for r in rows),
            "tokens": sum(r.get("supervised_tokens", 0) for r in rows), "update_seconds": sum(r["seconds"] for r in rows), "samples": len(rows),
            "mtime": path.stat().st_mtime}


@dataclass(frozen=True)
class Guard:
    min_free_gpu_gib: float = 55.0
    min_free_host_gib: float = 32.0
    stale_after_seconds: float = 300.0

    def reason(self, training_roots: dict[str, str], snapshot: dict[str, dict], free_gpu_gib: float, free_host_gib: float, now: float) -> str | None:
        if free_gpu_gib < self.min_free_gpu_gib:
            return f"GPU headroom below {self.min_free_gpu_gib:g} GiB"
        if free_host_gib < self.min_free_host_gib:
            return f"host headroom below {self.min_free_host_gib:g} GiB"
        if any(now - row["mtime"] > self.stale_after_seconds for row in snapshot.values()):
            return "trainer metrics stale"
        if any((Path(root) / "TRAINING_COMPLETE.json").exists() for root in training_roots.values()):
            return "yield before the training queue advances"
        return None


def stop_child(process: subprocess.Popen, grace: float = 30.0) -> None:
    """The child was started in a new session, so its pid is its process-group id; nothing else is ever signalled."""
    if process.poll() is None:
        os.killpg(process.pid, signal.SIGTERM)
        try:
            process.wait(timeout=grace)
        except subprocess.TimeoutExpired:
            os.killpg(process.pid, signal.SIGKILL)
            process.wait(timeout=grace)


class CoEvaluator:
    def __init__(self, output, training_roots: dict[str, str], *, free_gpu_gib: Callable[[], float], free_host_gib: Callable[[], float],
                 guard: Guard = Guard(), poll_seconds: float = 5.0, max_hours: float = 12.0, metrics_name: str = "train-metrics.jsonl",
                 clock: Callable[[], float] = time.time):
        self.output, self.roots, self.guard = Path(output), dict(training_roots), guard
        self.free_gpu, self.free_host, self.poll, self.max_seconds, self.metrics_name, self.clock = free_gpu_gib, free_host_gib, poll_seconds, max_hours * 3600, metrics_name, clock

    def _snapshot(self) -> dict[str, dict]:
        return {arm: tail_metrics(Path(root) / self.metrics_name) for arm, root in self.roots.items()}

    def run(self, phases: list[dict]) -> dict:
        """``phases``: ``[{"name": str, "command": [...], "env": {...}}]``.  Returns the queue receipt (also written)."""
        out = self.output
        out.mkdir(parents=True, exist_ok=True)
        if (out / "STOP").exists() or (out / "COMPLETE.json").exists():
            raise ValueError("the queue output is already stopped or complete")
        baseline = self._snapshot()
        atomic_write_json(out / "BASELINE.json", baseline)
        began, done = time.monotonic(), []
        for index, phase in enumerate(phases):
            log = (out / f"phase-{index}-{phase['name']}.log").open("wb")
            child = subprocess.Popen(phase["command"], env={**os.environ, **phase.get("env", {})}, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
            why = None
            try:
                while child.poll() is None:
                    if (out / "STOP").exists():
                        why = "STOP file"
                    elif time.monotonic() - began > self.max_seconds:
                        why = "queue time limit"
                    else:
                        why = self.guard.reason(self.roots, self._snapshot(), self.free_gpu(), self.free_host(), self.clock())
                    if why:
                        break
                    time.sleep(self.poll)
            finally:
                stop_child(child)
                log.close()
            now = self._snapshot()
            slowdown = {arm: now[arm]["median_seconds"] / baseline[arm]["median_seconds"] for arm in baseline}
            receipt = {"phase": phase["name"], "returncode": child.returncode, "yielded": why, "trainer_slowdown": slowdown, "trainer_step": {a: now[a]["step"] for a in now}}
            atomic_write_json(out / f"phase-{index}-{'YIELDED' if why else 'DONE'}.json", receipt)
            done.append(receipt)
            if why or child.returncode != 0:
                final = {"complete": False, "stopped_at": phase["name"], "reason": why or f"exit code {child.returncode}", "phases": done}
                atomic_write_json(out / "STOPPED.json", final)
                return final
        final = {"complete": True, "phases": done}
        atomic_write_json(out / "COMPLETE.json", final)
        return final
