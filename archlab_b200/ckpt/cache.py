"""Once-per-node, content-addressed staging of verified checkpoint payloads.

Several local ranks that resume from the same checkpoint on shared storage copy it once to node-local storage: the cache
entry is named by the SHA-256 of the checkpoint's ``COMPLETE.json`` receipt (``{"files": {name: sha256}}``), filled in a
private directory, verified file by file against the receipt and only then published with one rename, all under a
per-entry file lock.  A published entry carries ``VERIFIED.json`` with the size / mtime / inode of every payload at
verification time; a later caller re-checks those identities instead of re-hashing, so a payload modified after
verification is refused.  The source is never written to.  (The reference stages V4.1 checkpoints this way:
src/archlab/automodel/checkpoint_cache.py:20-66.)
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import shutil
import tempfile
from pathlib import Path

from ..contracts.substrate import atomic_write_json, sha256_file

RECEIPT, PROOF = "COMPLETE.json", "VERIFIED.json"


def _identity(path: Path) -> dict:
    st = path.stat()
    return {"size": st.st_size, "mtime_ns": st.st_mtime_ns, "inode": st.st_ino}


def _check_published(entry: Path, key: str, receipt_bytes: bytes, names: set[str]) -> Path:
    if (entry / RECEIPT).read_bytes() != receipt_bytes:
        raise ValueError("cached checkpoint receipt changed")
    proof = json.loads((entry / PROOF).read_text())
    if proof["receipt_sha256"] != key or set(proof["payloads"]) != names:
        raise ValueError("cached checkpoint verification differs from its receipt")
    for name, expected in proof["payloads"].items():
        if _identity(entry / name) != expected:
            raise ValueError("verified checkpoint payload changed: " + name)
    return entry


def stage_checkpoint(source, cache_root) -> Path:
    """Path of the verified node-local copy of ``source`` (copied by the first caller, shared by the others)."""
    source, cache_root = Path(source), Path(cache_root)
    receipt_bytes = (source / RECEIPT).read_bytes()
    files = json.loads(receipt_bytes)["files"]
    for name in files:
        if Path(name).name != name or name in (RECEIPT, PROOF):
            raise ValueError("checkpoint receipt contains an unsafe payload name")
    key = hashlib.sha256(receipt_bytes).hexdigest()
    cache_root.mkdir(parents=True, exist_ok=True)
    entry = cache_root / key
    with (cache_root / f"{key}.lock").open("a") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)                    # local ranks queue here; the first one copies
        if entry.exists():
            return _check_published(entry, key, receipt_bytes, set(files))
        scratch = Path(tempfile.mkdtemp(prefix=f"{key}.partial-", dir=cache_root))
        try:
            for name, digest in files.items():
                shutil.copyfile(source / name, scratch / name)
                if sha256_file(scratch / name) != digest:
                    raise ValueError("staged checkpoint checksum mismatch: " + name)
            if (source / RECEIPT).read_bytes() != receipt_bytes:
                raise ValueError("source checkpoint receipt changed during staging")
            (scratch / RECEIPT).write_bytes(receipt_bytes)
            atomic_write_json(scratch / PROOF, {"receipt_sha256": key, "source": str(source),
                                                "payloads": {name: _identity(scratch / name) for name in files}})
            scratch.rename(entry)                           # nothing partial is ever visible under the entry's name
        finally:
            if scratch.exists():
                shutil.rmtree(scratch)
    return entry
