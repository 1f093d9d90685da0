"""Storage hygiene: verified bulk offload with a SQLite journal (src/archlab/storage/bulk_offload.py:17-108).
Checkpoint retention is the service in ``services.retention``."""
from __future__ import annotations

import os
import shutil
import sqlite3
import time
from pathlib import Path

from ..contracts.substrate import sha256_file


def confined(root: Path, relative: str) -> Path:
    p = (root / relative).resolve()
    p.relative_to(root.resolve())                      # raises ValueError when it escapes
    return p


class OffloadJournal:
    def __init__(self, path):
        self.db = sqlite3.connect(str(path))
        self.db.execute("CREATE TABLE IF NOT EXISTS transfers (source TEXT PRIMARY KEY, destination TEXT, bytes INTEGER, "
                        "sha256 TEXT, state TEXT, updated REAL)")
        self.db.commit()

    def record(self, source, destination, nbytes, digest, state):
        self.db.execute("INSERT OR REPLACE INTO transfers VALUES (?, ?, ?, ?, ?, ?)",
                        (str(source), str(destination), nbytes, digest, state, time.time()))
        self.db.commit()

    def state(self, source):
        row = self.db.execute("SELECT state, sha256 FROM transfers WHERE source = ?", (str(source),)).fetchone()
        return row or (None, None)


def transfer(source, destination, journal: OffloadJournal, *, link: bool = False, expected_sha: str | None = None,
             delete_source: bool = False) -> dict:
    """Copy (or hard-link), re-hash the destination, journal the result; the source is removed only after
    the destination verified."""
    source, destination = Path(source), Path(destination)
    state, digest = journal.state(source)
    if state == "verified" and destination.is_file() and sha256_file(destination) == digest:
        return {"source": str(source), "state": "already-verified", "sha256": digest}
    src_sha = sha256_file(source)
    if expected_sha is not None and src_sha != expected_sha:
        raise ValueError(f"source content differs from the expected hash: {source}")
    destination.parent.mkdir(parents=True, exist_ok=True)
    tmp = destination.with_name(destination.name + ".partial")
    journal.record(source, destination, source.stat().st_size, src_sha, "copying")
    if link:
        tmp.unlink(missing_ok=True)
        os.link(source, tmp)
    else:
        shutil.copyfile(source, tmp)
    if sha256_file(tmp) != src_sha:
        tmp.unlink(missing_ok=True)
        journal.record(source, destination, source.stat().st_size, src_sha, "failed")
        raise RuntimeError(f"destination hash mismatch for {source}")
    tmp.replace(destination)
    journal.record(source, destination, destination.stat().st_size, src_sha, "verified")
    if delete_source:
        source.unlink()
    return {"source": str(source), "state": "verified", "sha256": src_sha}
