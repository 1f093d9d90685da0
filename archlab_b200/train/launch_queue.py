"""File-backed launch-request queue with a single consumer.

A requester drops ``requests/<generation>.json`` (written atomically) under a control directory; the
controller - one process, guarded by a lock file - validates every field against a closed schema,
proves that the named repository snapshot is the requested commit with a clean tree, runs the allowed
launcher with the validated environment, and records ``results/<generation>.json``.  A generation is
processed once: a request whose digest differs from the one already recorded is refused, never re-run.
Heartbeats and an append-only event log let an outside watcher tell "idle" from "dead".

Same contract as the reference's PAI-DLC controller (src/archlab/dlc_controller.py:136-691: exact-key
JSON, git-verified snapshot, single consumer); the schema here is data (``RequestSchema``) rather than
module constants so that tests and other clusters can supply their own roots and launchers.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import signal
import socket
import subprocess
import time
from dataclasses import dataclass, field
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Callable

SCHEMA_VERSION = 1
_GENERATION = re.compile(r"[A-Za-z0-9][A-Za-z0-9._-]{0,79}\Z")
_COMMIT = re.compile(r"[0-9a-f]{40}\Z")
_TOP = {"schema_version", "generation", "action", "requested_at_utc", "requested_from", "repository", "launcher", "environment"}


@dataclass(frozen=True)
class RequestSchema:
    launchers: frozenset[str]
    repo_root: Path
    requested_from: str
    allowed_env: frozenset[str]
    required_env: frozenset[str]
    positive_int: frozenset[str] = frozenset()
    nonnegative_int: frozenset[str] = frozenset()
    boolean: frozenset[str] = frozenset()
    choices: dict = field(default_factory=dict)              # key -> allowed values
    path_prefix: dict = field(default_factory=dict)          # key -> root the path must live under


@dataclass(frozen=True)
class LaunchRequest:
    generation: str
    repository_root: Path
    commit: str
    launcher: str
    environment: dict
    payload: dict
    digest: str


def canonical_json(payload: dict) -> bytes:
    return (json.dumps(payload, sort_keys=True, separators=(",", ":")) + "\n").encode()


def digest(payload: dict) -> str:
    return hashlib.sha256(canonical_json(payload)).hexdigest()


def utc_now() -> str:
    return datetime.now(timezone.utc).isoformat().replace("+00:00", "Z")


def _line(value: Any, label: str) -> str:
    if not isinstance(value, str) or not value or "\x00" in value or "\n" in value:
        raise ValueError(f"{label} must be a non-empty single-line string")
    return value


def _within(path: Path, root: Path) -> bool:
    try:
        path.resolve(strict=False).relative_to(root.resolve(strict=False))
        return True
    except ValueError:
        return False


def validate_request(payload: Any, schema: RequestSchema, *, expected_nodes: int | None = None,
                     expected_gpus_per_node: int | None = None, nodes_key: str = "NGA_EXPECTED_NODES",
                     gpus_key: str = "NGA_GPUS_PER_NODE") -> LaunchRequest:
    if not isinstance(payload, dict):
        raise ValueError("launch request must be a JSON object")
    if set(payload) - _TOP:
        raise ValueError(f"unsupported launch request keys: {sorted(set(payload) - _TOP)}")
    if _TOP - set(payload):
        raise ValueError(f"missing launch request keys: {sorted(_TOP - set(payload))}")
    if payload["schema_version"] != SCHEMA_VERSION:
        raise ValueError(f"schema_version must be {SCHEMA_VERSION}")
    if payload["action"] != "run":
        raise ValueError("action must be 'run'")
    generation = _line(payload["generation"], "generation")
    if not _GENERATION.fullmatch(generation):
        raise ValueError("generation contains unsupported characters")
    stamp = datetime.fromisoformat(_line(payload["requested_at_utc"], "requested_at_utc").replace("Z", "+00:00"))
    if stamp.tzinfo is None or stamp.utcoffset() != timezone.utc.utcoffset(stamp):
        raise ValueError("requested_at_utc must be a UTC timestamp")
    if _line(payload["requested_from"], "requested_from") != schema.requested_from:
        raise ValueError(f"requested_from must be {schema.requested_from}")
    launcher = _line(payload["launcher"], "launcher")
    if launcher not in schema.launchers:
        raise ValueError(f"launcher must be one of {sorted(schema.launchers)}")
    repo = payload["repository"]
    if not isinstance(repo, dict) or set(repo) != {"root", "commit"}:
        raise ValueError("repository must contain exactly root and commit")
    root = Path(_line(repo["root"], "repository.root"))
    if not root.is_absolute() or not _within(root, schema.repo_root):
        raise ValueError(f"repository.root must be under {schema.repo_root}")
    commit = _line(repo["commit"], "repository.commit")
    if not _COMMIT.fullmatch(commit):
        raise ValueError("repository.commit must be a full lowercase SHA-1")
    env_in = payload["environment"]
    if not isinstance(env_in, dict):
        raise ValueError("environment must be an object")
    if set(env_in) - schema.allowed_env:
        raise ValueError(f"unsupported environment keys: {sorted(set(env_in) - schema.allowed_env)}")
    if schema.required_env - set(env_in):
        raise ValueError(f"missing environment keys: {sorted(schema.required_env - set(env_in))}")
    env = {k: _line(v, f"environment.{k}") for k, v in env_in.items()}
    for k in schema.positive_int & set(env):
        if not env[k].isdigit() or int(env[k]) < 1:
            raise ValueError(f"{k} must be a positive integer")
    for k in schema.nonnegative_int & set(env):
        if not env[k].isdigit():
            raise ValueError(f"{k} must be a non-negative integer")
    for k in schema.boolean & set(env):
        if env[k] not in ("0", "1"):
            raise ValueError(f"{k} must be 0 or 1")
    for k, allowed in schema.choices.items():
        if k in env and env[k] not in allowed:
            raise ValueError(f"{k} must be one of {sorted(allowed)}")
    for k, prefix in schema.path_prefix.items():
        if k in env and (not Path(env[k]).is_absolute() or not _within(Path(env[k]), Path(prefix))):
            raise ValueError(f"{k} must be an absolute path under {prefix}")
    if expected_nodes is not None and int(env.get(nodes_key, -1)) != expected_nodes:
        raise ValueError(f"{nodes_key} must equal the controller's node count {expected_nodes}")
    if expected_gpus_per_node is not None and int(env.get(gpus_key, -1)) != expected_gpus_per_node:
        raise ValueError(f"{gpus_key} must equal the controller's GPUs per node {expected_gpus_per_node}")
    return LaunchRequest(generation, root, commit, launcher, env, payload, digest(payload))


def atomic_write_json(path: Path, payload: dict) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(f".{path.name}.{os.getpid()}.tmp")
    with open(tmp, "wb") as f:
        f.write(canonical_json(payload))
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _git(root: Path, *args: str) -> str:
    res = subprocess.run(["git", "-C", str(root), *args], capture_output=True, text=True)
    if res.returncode:
        raise RuntimeError(f"git {' '.join(args)} failed: {res.stderr.strip()}")
    return res.stdout.strip()


def verify_repository(request: LaunchRequest) -> None:
    """The snapshot must sit exactly at the requested commit, with nothing modified or untracked."""
    if _git(request.repository_root, "rev-parse", "HEAD") != request.commit:
        raise RuntimeError("repository HEAD does not match the requested commit")
    if _git(request.repository_root, "status", "--porcelain", "--untracked-files=all"):
        raise RuntimeError("repository snapshot has local modifications")
    if not (request.repository_root / request.launcher).is_file():
        raise RuntimeError("launcher is not part of the snapshot")


def publish_request(control_root: Path, payload: dict, schema: RequestSchema) -> Path:
    """Validate, then place the request where the controller looks; refuses to overwrite a generation."""
    req = validate_request(payload, schema)
    dst = Path(control_root) / "requests" / f"{req.generation}.json"
    if dst.exists():
        if digest(json.loads(dst.read_text())) != req.digest:
            raise FileExistsError(f"generation {req.generation} already published with different content")
        return dst
    atomic_write_json(dst, payload)
    return dst


class Controller:
    def __init__(self, control_root: Path, schema: RequestSchema, *, poll_seconds: float = 5.0, expected_nodes: int | None = None,
                 expected_gpus_per_node: int | None = None, runner: Callable | None = None, verify: Callable = verify_repository):
        self.root, self.schema, self.poll = Path(control_root), schema, poll_seconds
        self.nodes, self.gpus = expected_nodes, expected_gpus_per_node
        self.runner, self.verify = runner or self._subprocess_runner, verify
        self.stop = False
        for d in ("requests", "results", "logs"):
            (self.root / d).mkdir(parents=True, exist_ok=True)
        self._lock = None

    # -- single consumer -----------------------------------------------------------------------------
    def acquire(self) -> None:
        lock = self.root / "controller.lock"
        try:
            fd = os.open(lock, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
        except FileExistsError:
            owner = lock.read_text().strip()
            raise RuntimeError(f"another controller holds {lock}: {owner}") from None
        os.write(fd, f"{socket.gethostname()}:{os.getpid()}\n".encode())
        os.close(fd)
        self._lock = lock

    def release(self) -> None:
        if self._lock is not None:
            self._lock.unlink(missing_ok=True)
            self._lock = None

    def request_stop(self, *_):
        self.stop = True

    # -- records -------------------------------------------------------------------------------------
    def event(self, name: str, **fields) -> None:
        with open(self.root / "events.jsonl", "a") as f:
            f.write(json.dumps({"time_utc": utc_now(), "event": name, **fields}, sort_keys=True) + "\n")

    def heartbeat(self, state: str, **fields) -> None:
        atomic_write_json(self.root / "heartbeat.json", {"time_utc": utc_now(), "state": state, "host": socket.gethostname(),
                                                         "pid": os.getpid(), **fields})

    def result_path(self, generation: str) -> Path:
        return self.root / "results" / f"{generation}.json"

    def already_processed(self, req: LaunchRequest) -> bool:
        p = self.result_path(req.generation)
        if not p.exists():
            return False
        if json.loads(p.read_text()).get("request_sha256") != req.digest:
            raise RuntimeError(f"generation {req.generation} was processed with different content")
        return True

    def _subprocess_runner(self, req: LaunchRequest, log_path: Path) -> int:
        env = {**os.environ, **req.environment}
        with open(log_path, "ab") as log:
            proc = subprocess.Popen(["bash", str(req.repository_root / req.launcher)], cwd=req.repository_root, env=env,
                                    stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
            while proc.poll() is None:
                if self.stop:
                    os.killpg(proc.pid, signal.SIGTERM)
                self.heartbeat("running", generation=req.generation, child=proc.pid)
                time.sleep(min(self.poll, 1.0))
            return proc.returncode

    # -- loop ----------------------------------------------------------------------------------------
    def process(self, path: Path) -> str:
        """Handle one request file; returns 'done', 'failed', 'rejected' or 'skipped'."""
        try:
            req = validate_request(json.loads(path.read_text()), self.schema, expected_nodes=self.nodes,
                                   expected_gpus_per_node=self.gpus)
            if path.stem != req.generation:
                raise ValueError("file name does not match the generation")
        except (ValueError, json.JSONDecodeError) as e:
            self.event("rejected", file=path.name, reason=str(e))
            path.rename(path.with_suffix(".rejected"))
            return "rejected"
        if self.already_processed(req):
            return "skipped"
        started = utc_now()
        try:
            self.verify(req)
            self.event("started", generation=req.generation, request_sha256=req.digest)
            rc = self.runner(req, self.root / "logs" / f"{req.generation}.log")
            status = "done" if rc == 0 else "failed"
            detail = {"returncode": rc}
        except Exception as e:                               # verification or launch failure: recorded, not retried
            status, detail = "failed", {"error": f"{type(e).__name__}: {e}"}
        atomic_write_json(self.result_path(req.generation), {"generation": req.generation, "request_sha256": req.digest,
                                                             "status": status, "started_utc": started, "finished_utc": utc_now(),
                                                             **detail})
        self.event(status, generation=req.generation, **detail)
        return status

    def serve(self, *, max_polls: int | None = None) -> int:
        self.acquire()
        try:
            polls = 0
            while not self.stop and (max_polls is None or polls < max_polls):
                for path in sorted((self.root / "requests").glob("*.json")):
                    if self.stop:
                        break
                    self.process(path)
                self.heartbeat("idle")
                polls += 1
                if max_polls is None or polls < max_polls:
                    time.sleep(self.poll)
            return 0
        finally:
            self.release()
