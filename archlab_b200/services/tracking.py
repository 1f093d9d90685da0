"""Follow append-only JSONL metric ledgers and forward new rows exactly once to a tracking client
(MLflow-compatible ``log_metrics(run, step, values)`` object): a byte cursor per ledger persisted
atomically, a single-writer lock file, torn trailing lines left for the next pass
(src/archlab/tracking/mlflow_sync.py:23-285, process_status.py)."""
from __future__ import annotations

import json
import math
import os
import time
from pathlib import Path

from ..contracts.substrate import atomic_write_json


class SingleWriterLock:
    """``O_EXCL`` lock file holding the owner's pid; a stale lock (dead pid) is taken over."""

    def __init__(self, path):
        self.path = Path(path)

    def __enter__(self):
        while True:
            try:
                fd = os.open(self.path, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
                os.write(fd, str(os.getpid()).encode())
                os.close(fd)
                return self
            except FileExistsError:
                try:
                    pid = int(self.path.read_text() or 0)
                    os.kill(pid, 0)
                except (ValueError, ProcessLookupError, FileNotFoundError):
                    self.path.unlink(missing_ok=True)
                    continue
                except PermissionError:
                    pass
                raise RuntimeError(f"another writer holds {self.path}")

    def __exit__(self, *exc):
        self.path.unlink(missing_ok=True)


def point_values(row: dict) -> dict[str, float]:
    """Finite numeric fields of a ledger row (booleans and non-finite values are dropped)."""
    return {k: float(v) for k, v in row.items()
            if isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v) and k != "step"}


class LedgerSync:
    def __init__(self, client, state_path):
        self.client, self.state_path = client, Path(state_path)
        self.state = json.loads(self.state_path.read_text()) if self.state_path.is_file() else {"cursors": {}}

    def sync(self, run: str, ledger) -> int:
        ledger = Path(ledger)
        key = str(ledger)
        pos = int(self.state["cursors"].get(key, 0))
        sent = 0
        with open(ledger, "rb") as f:
            f.seek(pos)
            while True:
                line = f.readline()
                if not line or not line.endswith(b"\n"):
                    break                                   # torn tail: retry next pass
                pos = f.tell()
                try:
                    row = json.loads(line)
                except json.JSONDecodeError:
                    continue
                vals = point_values(row)
                if vals:
                    self.client.log_metrics(run, int(row.get("step", 0)), vals)
                    sent += 1
        self.state["cursors"][key] = pos
        atomic_write_json(self.state_path, self.state)
        return sent


def process_status(pid_file, heartbeat_file, *, stale_after: float = 300.0, now: float | None = None) -> dict:
    """RUNNING / STALLED / EXITED from a pid file and a heartbeat file's mtime."""
    now = time.time() if now is None else now
    try:
        pid = int(Path(pid_file).read_text())
        os.kill(pid, 0)
        alive = True
    except (ValueError, FileNotFoundError, ProcessLookupError):
        alive, pid = False, None
    except PermissionError:
        alive = True
    age = now - Path(heartbeat_file).stat().st_mtime if Path(heartbeat_file).exists() else math.inf
    state = "EXITED" if not alive else ("STALLED" if age > stale_after else "RUNNING")
    return {"state": state, "pid": pid, "heartbeat_age_s": age}
