"""Runtime substrate: atomic JSON publication, file identities, failure taxonomy.

Counterparts in the reference: src/archlab/artifacts.py:17-76 (``atomic_write_json``,
``sha256_file``, ``transfer_plan``) and src/archlab/failures.py:18-47 (``classify_failure``).
"""
from __future__ import annotations

import hashlib
import json
import os
import tempfile
from dataclasses import asdict, dataclass
from pathlib import Path, PurePosixPath
from typing import Any


def sha256_file(path: str | Path, *, chunk_bytes: int = 8 << 20) -> str:
    if chunk_bytes < 1:
        raise ValueError("hash chunk size must be positive")
    h = hashlib.sha256()
    with Path(path).open("rb") as f:
        for chunk in iter(lambda: f.read(chunk_bytes), b""):
            h.update(chunk)
    return h.hexdigest()


def canonical_json(payload: Any) -> str:
    return json.dumps(payload, sort_keys=True, separators=(",", ":"), ensure_ascii=True)


def sha256_json(payload: Any) -> str:
    return hashlib.sha256(canonical_json(payload).encode()).hexdigest()


def atomic_write_json(path: str | Path, payload: Any, *, ensure_ascii: bool = True, allow_nan: bool = True,
                      create_parents: bool = True, sort_keys: bool = True) -> None:
    """Indented JSON + LF written to a temporary file in the same directory, fsynced, then renamed
    over the target: readers see the old file or the new one, never a torn write."""
    path = Path(path)
    if create_parents:
        path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=f".{path.name}.", suffix=".tmp", dir=path.parent)
    try:
        with os.fdopen(fd, "w", encoding="utf-8", newline="\n") as f:
            json.dump(payload, f, indent=2, sort_keys=sort_keys, ensure_ascii=ensure_ascii, allow_nan=allow_nan)
            f.write("\n")
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)


def atomic_write_bytes(path: str | Path, data: bytes) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=f".{path.name}.", suffix=".tmp", dir=path.parent)
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)


def transfer_plan(source: str | Path, destination: str) -> tuple[list[PurePosixPath], list[tuple[Path, str]]]:
    """Directories to create and (local file, remote path) pairs for uploading a file or a tree;
    links and special files are rejected before anything is transferred."""
    source = Path(source)
    if source.is_file():
        return [], [(source, destination + source.name if destination.endswith("/") else destination)]
    if not source.is_dir() or source.is_symlink():
        raise ValueError("transfer source must be a file or regular directory")
    entries = sorted(source.rglob("*"))
    if any(p.is_symlink() or not (p.is_file() or p.is_dir()) for p in entries):
        raise ValueError("directory transfer supports regular files and directories only")
    root = PurePosixPath(destination)
    dirs = [root, *(root / p.relative_to(source) for p in entries if p.is_dir())]
    files = [(p, str(root / p.relative_to(source))) for p in entries if p.is_file()]
    return dirs, files


@dataclass(frozen=True)
class FailureClassification:
    category: str       # numerical | capacity | operational | contract | unknown
    retriable: bool
    reason: str

    def to_dict(self) -> dict:
        return asdict(self)


_NUMERICAL = ("non-finite", "nan", "infinity", "inf gradient")
_CAPACITY = ("out of memory", "cuda oom", "cublas_status_alloc")
_OPERATIONAL = ("nccl", "connection reset", "connection closed", "timed out", "timeout", "preempt", "sigterm",
                "temporary failure", "device status word")
_CONTRACT = ("contract", "manifest", "mismatch", "missing", "refusing to overwrite")


def classify_failure(error: BaseException) -> FailureClassification:
    """Conservative triage: only transient infrastructure failures may be retried unchanged.  A
    device status word raised by a bounded in-kernel wait counts as operational."""
    msg = f"{type(error).__name__}: {error}".lower()
    if any(t in msg for t in _NUMERICAL):
        return FailureClassification("numerical", False, "non-finite model state or metric")
    if any(t in msg for t in _CAPACITY):
        return FailureClassification("capacity", False, "the declared configuration exceeds capacity")
    if any(t in msg for t in _OPERATIONAL):
        return FailureClassification("operational", True, "transient infrastructure failure")
    if isinstance(error, (ValueError, AssertionError, FileNotFoundError)) or any(t in msg for t in _CONTRACT):
        return FailureClassification("contract", False, "experiment precondition failed")
    return FailureClassification("unknown", False, "manual triage required before retry")
