"""Follow append-only JSONL metric ledgers and forward new rows exactly once to a tracking client
(MLflow-compatible ``log_metrics(run, step, values)`` object): a byte cursor per ledger persisted
atomically, a single-writer lock file, torn trailing lines left for the next pass
(src/archlab/tracking/mlflow_sync.py:23-285, process_status.py)."""
from __future__ import annotations

import hashlib
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


# ======================================================================================================================
# Run-level sync: training ledgers of registered runs -> a tracking store, exactly once, resumable after any crash.
#
# What the reference's MLflow follower guarantees (src/archlab/tracking/mlflow_sync.py:200-547) and this one keeps:
#   * a run is identified by its *source id* (never by name); two store runs with one source id are refused;
#   * the ledger must be contiguous (step + 1, token cursor + tokens of the row) and finite before anything is sent;
#   * the step cursor lives in a local state file; a cursor ahead of the ledger is refused (a ledger was replaced);
#   * points go out in bounded batches whose timestamp is chosen and persisted BEFORE the write, so a retry after a crash
#     re-sends the same points with the same timestamp (stores de-duplicate identical points);
#   * a change of the source commit under a live run needs a qualified ``SOURCE_TRANSITION.json`` (from / to commit,
#     ``training_math_unchanged``, cursor not behind what was sent); otherwise histories would silently be mixed;
#   * validation rows are keyed to the training token cursor and sent once per content fingerprint.
# The store is any object with the five methods of ``FileTrackingStore``; an MLflow client adapter maps them to
# ``search_runs`` / ``create_run`` / ``log_batch``.
BATCH_POINTS = 60
TRAIN_METRICS = {"train/cross_entropy": "loss", "train/supervised_tokens": "consumed_supervised_tokens",
                 "optim/learning_rate": "learning_rate", "optim/gradient_norm": "gradient_norm_before_clip",
                 "memory/peak_allocated_gib": "max_memory_allocated_gib", "router/load_cv": "router_load_cv_mean",
                 "router/unused_fraction": "router_unused_fraction_window"}
REQUIRED_FIELDS = ("step", "loss", "supervised_tokens", "consumed_supervised_tokens")


def read_contiguous_ledger(paths) -> list[dict]:
    """Complete rows of one or more ledger files in order; an unterminated last line belongs to a live writer."""
    rows = []
    for path in paths:
        body = Path(path).read_text()
        rows += [json.loads(line) for line in body.split("\n")[:-1] if line.strip()]
    if not rows:
        raise ValueError("no complete training records")
    for before, row in zip([None, *rows], rows):
        if any(k not in row for k in REQUIRED_FIELDS) or not math.isfinite(row["loss"]) or row["supervised_tokens"] <= 0:
            raise ValueError(f"invalid training record at step {row.get('step')}")
        if before is not None and (row["step"] != before["step"] + 1 or
                                   row["consumed_supervised_tokens"] != before["consumed_supervised_tokens"] + row["supervised_tokens"]):
            raise ValueError(f"training ledger is not contiguous at step {row['step']}")
    return rows


def training_points(row: dict) -> dict[str, float]:
    seconds = row.get("wall_seconds", row.get("seconds", row.get("step_seconds")))
    if seconds is None or seconds <= 0:
        raise ValueError("nonpositive update duration")
    out = {name: float(row[key]) for name, key in TRAIN_METRICS.items() if key in row and row[key] is not None}
    out["perf/target_tokens_per_second"] = row["supervised_tokens"] / seconds
    out["perf/seconds_per_update"] = float(seconds)
    return out


class FileTrackingStore:
    """Offline tracking store: one directory per run with ``meta.json`` and an append-only ``points.jsonl``.
    Identical points (name, axis value, value, timestamp) are stored once, like a tracking server does."""

    def __init__(self, root):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)

    def find_runs(self, source_id: str) -> list[str]:
        return sorted(p.parent.name for p in self.root.glob("*/meta.json") if json.loads(p.read_text())["source_id"] == source_id)

    def create_run(self, source_id: str, name: str, tags: dict) -> str:
        run_id = f"{len(list(self.root.glob('*/meta.json'))):04d}-{name}"
        atomic_write_json(self.root / run_id / "meta.json", {"source_id": source_id, "name": name, "tags": tags, "params": {}})
        return run_id

    def set_fields(self, run_id: str, *, params: dict | None = None, tags: dict | None = None) -> None:
        meta = json.loads((self.root / run_id / "meta.json").read_text())
        meta["params"].update({k: str(v) for k, v in (params or {}).items()})
        meta["tags"].update(tags or {})
        atomic_write_json(self.root / run_id / "meta.json", meta)

    def log_points(self, run_id: str, points: list[tuple[str, float, int, int]]) -> None:
        """``(metric, value, axis value, timestamp ms)``."""
        path = self.root / run_id / "points.jsonl"
        seen = {line for line in path.read_text().splitlines()} if path.exists() else set()
        fresh = [line for line in (json.dumps(list(p)) for p in points) if line not in seen]
        with path.open("a") as f:
            f.writelines(line + "\n" for line in dict.fromkeys(fresh))

    def last_axis_value(self, run_id: str, metric: str) -> int | None:
        path = self.root / run_id / "points.jsonl"
        steps = [p[2] for p in map(json.loads, path.read_text().splitlines()) if p[0] == metric] if path.exists() else []
        return max(steps, default=None)


class TrackingSync:
    def __init__(self, store, state_path, *, clock=time.time):
        self.store, self.state_path, self.clock = store, Path(state_path), clock
        self.state = json.loads(self.state_path.read_text()) if self.state_path.exists() else {"runs": {}}

    def _save(self) -> None:
        atomic_write_json(self.state_path, self.state, sort_keys=False)

    def _ms(self) -> int:
        return int(self.clock() * 1000)

    # ---- identity ------------------------------------------------------------------------------------------------
    def _adopt_source_change(self, local: dict, spec: dict, commit: str) -> None:
        note = Path(spec["path"]) / "SOURCE_TRANSITION.json"
        change = json.loads(note.read_text()) if note.is_file() else {}
        qualified = (change.get("from_commit") == local["source_commit"] and change.get("to_commit") == commit
                     and change.get("training_math_unchanged") is True
                     and change.get("cursor", {}).get("step", -1) >= (local["last_step"] or 0))
        if not qualified:
            raise ValueError("existing tracking run source changed without a qualified continuation")
        local["source_history"] = [*local.get("source_history", []), local["source_commit"]]
        local["source_commit"] = commit
        self.store.set_fields(local["run_id"], tags={"archlab.current_source_commit": commit,
                                                     "archlab.prior_source_commits": json.dumps(local["source_history"])})
        self._save()

    def ensure_run(self, spec: dict, contract: dict) -> dict:
        commit = contract["project_commit"]
        local = self.state["runs"].get(spec["id"])
        if local is not None:
            if local["source_commit"] != commit:
                self._adopt_source_change(local, spec, commit)
            return local
        known = self.store.find_runs(spec["id"])
        if len(known) > 1:
            raise ValueError("duplicate tracking run identities")
        run_id = known[0] if known else self.store.create_run(spec["id"], spec["name"], {
            "archlab_source_id": spec["id"], "archlab.phase": spec.get("phase"), "archlab.variant": spec.get("variant"),
            "archlab.history_timestamps": "ingestion, not original wall-clock time"})
        local = {"run_id": run_id, "source_commit": commit, "history_timestamp_ms": self._ms(), "aux_fingerprints": {},
                 "last_step": self.store.last_axis_value(run_id, "train/cross_entropy") if known else None}
        params = {"variant": spec.get("variant"), "phase": spec.get("phase"), "gpu_type": "NVIDIA B200", "gpus": contract.get("world_size"),
                  "source_commit": commit, "optimizer": contract.get("optimizer"), "dataset": spec.get("dataset"),
                  "target_supervised_tokens": spec.get("budget"), "precision": (contract.get("precision") or {}).get("recipe"),
                  "timestamp_semantics": "ingestion time; optimizer-step and token axes are exact"}
        self.store.set_fields(run_id, params={k: v for k, v in params.items() if v is not None})
        self.state["runs"][spec["id"]] = local
        self._save()
        return local

    # ---- one run -------------------------------------------------------------------------------------------------
    def sync_run(self, spec: dict) -> dict:
        root = Path(spec["path"])
        history = spec.get("history") or [root / "train-metrics.jsonl"]
        if spec.get("defer_until_training") and not any(Path(p).is_file() for p in history):
            return {"id": spec["id"], "state": "queued", "new_updates": 0}
        contract = json.loads((root / "RUN_CONTRACT.json").read_text())
        rows = read_contiguous_ledger(history)
        local = self.ensure_run(spec, contract)
        if local["last_step"] is not None and local["last_step"] > rows[-1]["step"]:
            raise ValueError("tracking cursor is ahead of source")
        todo = [r for r in rows if local["last_step"] is None or r["step"] > local["last_step"]]
        backfill = len(todo) > BATCH_POINTS
        for i in range(0, len(todo), BATCH_POINTS):
            batch = todo[i:i + BATCH_POINTS]
            planned = local.get("pending_batch") or {}
            if planned.get("first_step") != batch[0]["step"]:           # choose the timestamp once, before the write
                planned = {"first_step": batch[0]["step"], "timestamp_ms": local["history_timestamp_ms"] if backfill else self._ms()}
                local["pending_batch"] = planned
                self._save()
            stamp = planned["timestamp_ms"]
            points = [(name, value, row["step"], stamp) for row in batch for name, value in training_points(row).items()]
            points += [("train/cross_entropy_by_tokens", float(row["loss"]), row["consumed_supervised_tokens"], stamp) for row in batch]
            self.store.log_points(local["run_id"], points)
            local["last_step"] = batch[-1]["step"]
            local.pop("pending_batch", None)
            self._save()
        sent_eval = self._sync_validation(root, rows, local)
        return {"id": spec["id"], "state": "synced", "new_updates": len(todo), "last_step": local["last_step"], "validation_points": sent_eval}

    def _sync_validation(self, root: Path, rows: list[dict], local: dict) -> int:
        ledger = root / "validation.jsonl"
        if not ledger.exists():
            return 0
        tokens_at = {r["step"]: r["consumed_supervised_tokens"] for r in rows}
        points = []
        for r in (json.loads(line) for line in ledger.read_text().split("\n")[:-1] if line.strip()):
            at = tokens_at.get(r["step"], 0 if r["step"] == 0 else None)      # an initial evaluation precedes any update
            if at is None:
                raise KeyError(f"validation step {r['step']} has no training token cursor")
            points += [("eval/cross_entropy", float(r["loss"]), r["step"]), ("eval/cross_entropy_by_tokens", float(r["loss"]), at)]
        digest = hashlib.sha256(json.dumps(points, sort_keys=True).encode()).hexdigest()
        if not points or local["aux_fingerprints"].get("validation") == digest:
            return 0
        stamp = local["history_timestamp_ms"]
        self.store.log_points(local["run_id"], [(*p, stamp) for p in points])
        local["aux_fingerprints"]["validation"] = digest
        self._save()
        return len(points)

    def sync_all(self, specs: list[dict]) -> dict:
        out = {"runs": [], "errors": []}
        for spec in specs:
            try:
                out["runs"].append(self.sync_run(spec))
            except Exception as error:                                 # one broken run must not starve the others
                out["errors"].append({"id": spec.get("id"), "error": f"{type(error).__name__}: {error}"})
        return out


def main(argv=None) -> int:
    import argparse
    import fcntl

    ap = argparse.ArgumentParser(description="Follow registered training ledgers into a tracking store.")
    ap.add_argument("--registry", type=Path, required=True, help="JSON list of run specs: id, name, path, [history, phase, variant, ...]")
    ap.add_argument("--store", type=Path, required=True, help="directory of the file tracking store")
    ap.add_argument("--state", type=Path, required=True)
    ap.add_argument("--watch", action="store_true")
    ap.add_argument("--interval", type=float, default=30.0)
    a = ap.parse_args(argv)
    a.state.parent.mkdir(parents=True, exist_ok=True)
    with open(str(a.state) + ".lock", "w") as lock:
        try:
            fcntl.flock(lock, fcntl.LOCK_EX | fcntl.LOCK_NB)           # one writer per state file
        except BlockingIOError:
            print("another tracking sync owns this state file", flush=True)
            return 0
        sync = TrackingSync(FileTrackingStore(a.store), a.state)
        while True:
            result = sync.sync_all(json.loads(a.registry.read_text()))
            print(json.dumps(result), flush=True)
            if not a.watch:
                return 1 if result["errors"] else 0
            time.sleep(a.interval)


if __name__ == "__main__":
    raise SystemExit(main())
