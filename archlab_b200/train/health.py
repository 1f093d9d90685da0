"""Run health: failure detection, graceful stop and liveness, all decided on the host.

* ``FiniteGuard``       - the step's loss (and optionally the gradient norm) must be finite on EVERY rank:
                          one MAX all-reduce of a flag per step; a non-finite value raises ``FloatingPointError``
                          on all ranks together (src/archlab/speedrun/base_train.py:810-880).
* ``StopConsensus``     - SIGTERM / SIGINT or a ``STOP_REQUESTED.json`` in the run directory raise a local flag;
                          the flag is MAX-reduced so that every rank leaves the loop at the SAME step, after which
                          the caller checkpoints and ``acknowledge`` writes ``STOPPED.json``
                          (src/archlab/megatron/simplicial_pilot.py:340-346,440-461).
* ``Heartbeat``         - ``HEARTBEAT.json`` rewritten at most every ``period`` seconds, also from inside long
                          accumulation steps, so that an outside watcher tells slow from dead (:397-402).
* ``collective_probe``  - a tiny all-reduce under a short timeout BEFORE training: a rank that never joins or a
                          broken fabric fails fast instead of hanging the first real collective
                          (src/archlab/collective_probe.py:40-62).
* ``assert_ranks_agree``- cross-rank equality of a digest (data cursor, weights after load): catches ranks that
                          silently diverged (simplicial_pilot.py:66-78).
Nothing here touches a GPU beyond the collectives the backend runs; waits are bounded by the process-group
timeout, and a missing rank surfaces as an exception classified "operational".
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import signal
import time
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist


def _dist() -> bool:
    return dist.is_available() and dist.is_initialized()


def _flag_max(value: float, device, group=None) -> float:
    t = torch.tensor([value], dtype=torch.float32, device=device)
    if _dist():
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


class FiniteGuard:
    def __init__(self, device="cpu", group=None):
        self.device, self.group = device, group

    def check(self, step: int, loss: float, grad_norm: float | None = None) -> None:
        bad = 0.0 if (math.isfinite(loss) and (grad_norm is None or math.isfinite(grad_norm))) else 1.0
        if _flag_max(bad, self.device, self.group) > 0:
            raise FloatingPointError(f"non-finite loss or gradient on some rank at step {step} (local loss {loss})")


class StopConsensus:
    def __init__(self, run_dir: Path, device="cpu", group=None, install_signals: bool = True):
        self.dir, self.device, self.group = Path(run_dir), device, group
        self.requested = False
        self.reason = None
        if install_signals:
            for sig in (signal.SIGTERM, signal.SIGINT):
                try:
                    signal.signal(sig, self._on_signal)
                except ValueError:                           # not the main thread
                    pass

    def _on_signal(self, signum, _frame):
        self.requested, self.reason = True, f"signal {signum}"

    def should_stop(self) -> bool:
        """Collective: call on every rank once per step."""
        if not self.requested and (self.dir / "STOP_REQUESTED.json").exists():
            self.requested, self.reason = True, "STOP_REQUESTED.json"
        return _flag_max(1.0 if self.requested else 0.0, self.device, self.group) > 0

    def acknowledge(self, step: int, rank: int = 0) -> None:
        if rank == 0:
            tmp = self.dir / ".STOPPED.json.tmp"
            tmp.write_text(json.dumps({"step": step, "reason": self.reason or "requested on another rank", "time": time.time()}))
            os.replace(tmp, self.dir / "STOPPED.json")


class Heartbeat:
    def __init__(self, run_dir: Path, period: float = 45.0, rank: int = 0):
        self.path, self.period, self.rank, self._last = Path(run_dir) / "HEARTBEAT.json", period, rank, 0.0

    def beat(self, **fields) -> bool:
        now = time.time()
        if self.rank != 0 or now - self._last < self.period:
            return False
        tmp = self.path.with_name(".HEARTBEAT.json.tmp")
        tmp.write_text(json.dumps({"time": now, "pid": os.getpid(), **fields}))
        os.replace(tmp, self.path)
        self._last = now
        return True


def collective_probe(device="cpu", *, timeout_seconds: float = 300.0) -> dict:
    """All ranks add 1; the sum must equal the world size.  Runs in its own short-timeout group so that an absent
    rank raises here (after ``timeout_seconds``) rather than wedging the trainer's first collective."""
    if not _dist():
        return {"world_size": 1, "seconds": 0.0}
    t0 = time.perf_counter()
    group = dist.new_group(timeout=timedelta(seconds=timeout_seconds))
    t = torch.ones(1, device=device)
    dist.all_reduce(t, group=group)
    if device != "cpu" and str(device).startswith("cuda"):
        torch.cuda.synchronize()
    if int(t.item()) != dist.get_world_size():
        raise RuntimeError(f"collective probe summed to {int(t.item())}, expected {dist.get_world_size()}")
    return {"world_size": dist.get_world_size(), "seconds": time.perf_counter() - t0}


def digest_tensors(tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.detach().to("cpu", torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


def assert_ranks_agree(label: str, digest: str, group=None) -> None:
    """Raises on every rank when any rank's digest differs from rank 0's."""
    if not _dist():
        return
    world = dist.get_world_size(group)
    got = [None] * world
    dist.all_gather_object(got, digest, group=group)
    if any(g != got[0] for g in got):
        raise RuntimeError(f"ranks disagree on {label}: {[g[:12] for g in got]}")
