"""Moving bulk payloads off the primary file system without ever having a moment where the data exists only half-way.

``offload_plan(source, destination)`` walks a results tree and lists the payload files worth moving (by suffix and size),
leaving alone: version-controlled directories, trees that declare active readers (``.archlab-storage-in-use.json``),
checkpoints without their completion marker, symlinks and retention tombstones.  Metadata stays where it is.

``TreeMigration`` moves one directory (a model, a dataset) in two explicit phases with a JSON journal:

* ``prepare``: inventory (regular files and directories only), copy every file with ``O_EXCL`` + fsync while hashing,
  re-hash the destination, reuse byte-identical files that are already there, refuse collisions, refuse a source that
  changed meanwhile; journal phase ``verified``.
* ``commit``: re-check source and destination against the journal, then replace the directory by a symlink to the copy.
  A directory and a symlink cannot be exchanged atomically on every file system, so the original is first renamed to a
  hidden backup; if publishing the link fails the backup is renamed back; the backup is deleted only after the path
  resolves to the verified copy and the backup itself is still unchanged.
(Reference: src/archlab/storage/model_migration.py:25-168, results_plan.py:10-43, bulk_offload.py:27-35.)
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import stat
import time
from pathlib import Path

from ..contracts.substrate import atomic_write_json, sha256_file

PAYLOAD_SUFFIXES = {".pt", ".pth", ".safetensors", ".bin", ".idx", ".npy", ".npz", ".arrow", ".parquet", ".gguf", ".u32", ".u16"}
IN_USE_MARKER = ".archlab-storage-in-use.json"


def assert_not_in_use(path) -> None:
    """Replacing files under readers on other clients is not safe; a guard file anywhere above the path forbids it."""
    for parent in Path(path).absolute().parents:
        readers = parent / ".checkpoint-readers"
        if (parent / IN_USE_MARKER).exists() or (readers.is_dir() and any(readers.glob("*.json"))):
            raise ValueError(f"active readers protect this storage tree: {parent}")


def offload_plan(source, destination, *, minimum_bytes: int = 4 << 20) -> tuple[list[dict], dict]:
    source, destination = Path(source).absolute(), Path(destination).absolute()
    tasks, pending, repositories, active = [], [], 0, []
    stack = [source]
    while stack:
        folder = stack.pop()
        with os.scandir(folder) as scan:
            entries = sorted(scan, key=lambda e: e.name)
        names = {e.name for e in entries}
        if IN_USE_MARKER in names:
            active.append(str(folder))
        elif ".git" in names:
            repositories += 1
        elif folder.name.startswith("step-") and folder.parent.name == "checkpoints" and "COMPLETE.json" not in names:
            pending.append(str(folder))
        else:
            for e in entries:
                if e.is_symlink():
                    continue
                if e.is_dir(follow_symlinks=False):
                    if not e.name.startswith(".retention-delete-"):
                        stack.append(Path(e.path))
                elif e.is_file(follow_symlinks=False) and Path(e.name).suffix.lower() in PAYLOAD_SUFFIXES:
                    size = e.stat(follow_symlinks=False).st_size
                    if size >= minimum_bytes:
                        rel = Path(e.path).relative_to(source)
                        tasks.append({"source": e.path, "destination": str(destination / rel), "bytes": size, "link": True})
    tasks.sort(key=lambda t: t["source"])
    return tasks, {"files": len(tasks), "bytes": sum(t["bytes"] for t in tasks), "incomplete_checkpoints_skipped": sorted(pending),
                   "repositories_skipped": repositories, "active_reader_trees_skipped": sorted(active), "minimum_bytes": minimum_bytes}


def tree_inventory(root: Path) -> dict[str, dict]:
    if root.is_symlink() or not root.is_dir():
        raise ValueError("the source must be a real directory")
    files = {}
    for parent, dirs, names in os.walk(root, followlinks=False):
        for name in dirs + names:
            path = Path(parent) / name
            info = path.lstat()
            if not (stat.S_ISREG(info.st_mode) or stat.S_ISDIR(info.st_mode)):
                raise ValueError(f"unsupported source entry: {path}")
            if stat.S_ISREG(info.st_mode):
                files[str(path.relative_to(root))] = {"bytes": info.st_size, "mtime_ns": info.st_mtime_ns, "inode": info.st_ino}
    return files


def _target(destination: Path, relative: str) -> Path:
    path = destination / relative
    for p in (path, *path.parents):
        if p.is_symlink():
            raise ValueError(f"a destination symlink would redirect a write: {p}")
        if p == destination:
            break
    return path


class TreeMigration:
    def __init__(self, journal):
        self.journal = Path(journal)

    def _save(self, state: dict) -> None:
        self.journal.parent.mkdir(parents=True, exist_ok=True)
        atomic_write_json(self.journal, state)

    def state(self) -> dict:
        return json.loads(self.journal.read_text())

    def prepare(self, source, destination) -> dict:
        source, destination = Path(source).absolute(), Path(destination).absolute()
        if source == destination or source in destination.parents or destination in source.parents:
            raise ValueError("source and destination must be disjoint")
        if destination.is_symlink() or not destination.is_dir():
            raise ValueError("the destination must already exist as a real directory")
        assert_not_in_use(source)
        files = tree_inventory(source)
        before = sorted(p.name for p in destination.iterdir())
        state = {"source": str(source), "destination": str(destination), "phase": "copying", "started": time.time(),
                 "destination_children_before": before, "files": {k: dict(v) for k, v in files.items()}, "bytes": sum(v["bytes"] for v in files.values())}
        self._save(state)
        for relative, info in files.items():
            src, dst = source / relative, _target(destination, relative)
            if dst.exists():
                if not dst.is_file() or dst.stat().st_size != info["bytes"] or sha256_file(dst) != sha256_file(src):
                    raise ValueError(f"destination collision: {relative}")
                state["files"][relative].update(sha256=sha256_file(dst), reused_existing=True)
            else:
                dst.parent.mkdir(parents=True, exist_ok=True)
                digest = hashlib.sha256()
                with src.open("rb") as fin, dst.open("xb") as fout:
                    while block := fin.read(8 << 20):
                        fout.write(block)
                        digest.update(block)
                    fout.flush()
                    os.fsync(fout.fileno())
                now = src.stat()
                if now.st_size != info["bytes"] or now.st_mtime_ns != info["mtime_ns"]:
                    raise ValueError(f"source changed during the copy: {relative}")
                if dst.stat().st_size != info["bytes"] or sha256_file(dst) != digest.hexdigest():
                    raise ValueError(f"destination verification failed: {relative}")
                state["files"][relative].update(sha256=digest.hexdigest(), reused_existing=False)
            self._save(state)
        if tree_inventory(source) != files:
            raise ValueError("the source tree changed during the migration")
        if not set(before) <= {p.name for p in destination.iterdir()}:
            raise ValueError("existing destination entries disappeared")
        state.update(phase="verified", verified=time.time())
        self._save(state)
        return state

    def commit(self, *, after_backup=None) -> dict:
        """``after_backup`` (tests): called between the two renames, to exercise the restore path."""
        state = self.state()
        if state["phase"] != "verified":
            raise ValueError("only a fully verified copy can be committed")
        source, destination = Path(state["source"]), Path(state["destination"])
        expected = {k: {n: v[n] for n in ("bytes", "mtime_ns", "inode")} for k, v in state["files"].items()}
        if tree_inventory(source) != expected:
            raise ValueError("the source changed after verification")
        for relative, info in state["files"].items():
            dst = _target(destination, relative)
            if dst.stat().st_size != info["bytes"] or sha256_file(dst) != info["sha256"]:
                raise ValueError(f"the verified destination changed: {relative}")
        tag = time.strftime("%Y%m%dT%H%M%SZ", time.gmtime())
        backup, link = source.parent / f".{source.name}.backup-{tag}", source.parent / f".{source.name}.link-{tag}"
        if backup.exists() or link.exists() or link.is_symlink():
            raise ValueError("a migration staging path exists")
        link.symlink_to(destination, target_is_directory=True)
        state.update(phase="switch_prepared", backup=str(backup), temporary_link=str(link))
        self._save(state)
        source.rename(backup)
        try:
            if after_backup is not None:
                after_backup()
            link.rename(source)
        except BaseException:
            backup.rename(source)                                   # the original is back where it was
            link.unlink(missing_ok=True)
            state.update(phase="verified")
            self._save(state)
            raise
        if not source.is_symlink() or source.resolve() != destination.resolve():
            raise ValueError("the link does not resolve to the verified destination")
        if any((source / r).stat().st_size != i["bytes"] for r, i in state["files"].items()):
            raise ValueError("the original path does not resolve correctly")
        if tree_inventory(backup) != expected:
            raise ValueError("the backup changed; it is kept for recovery")
        state.update(phase="linked", linked=time.time())
        self._save(state)
        shutil.rmtree(backup)
        state.update(phase="complete", completed=time.time(), removed_bytes=state["bytes"])
        self._save(state)
        return state


# ---- continuing offload as new finished payloads appear ----------------------------------------------------------------
def grow_plan(plan_path, candidates: list[dict]) -> int:
    """Adds tasks whose source is not in the plan yet (existing rows, with whatever state they carry, are kept);
    the plan file is replaced atomically.  Returns how many were added."""
    plan_path = Path(plan_path)
    known = {}
    if plan_path.exists():
        known = {row["source"]: row for row in (json.loads(line) for line in plan_path.read_text().splitlines() if line.strip())}
    added = 0
    for row in candidates:
        if row["source"] not in known:
            known[row["source"]] = row
            added += 1
    if added:
        tmp = plan_path.with_suffix(".tmp")
        tmp.write_text("".join(json.dumps(r) + "\n" for r in known.values()))
        tmp.replace(plan_path)
    return added


def offload_watch(source, destination, plan_path, journal_path, *, cycles: int | None = None, sleep_seconds: float = 120.0, minimum_bytes: int = 4 << 20,
                  sleep=time.sleep) -> dict:
    """Every cycle: re-plan the tree, append new finished payloads to the plan, transfer what the journal has not verified
    yet (``services.storage.transfer``: copy, re-hash, journal), write the status file beside the journal.  A transfer
    error stops the watcher with the status saying so -- nothing is retried blindly.  ``cycles=None`` runs until
    interrupted.  (Reference: src/archlab/storage/offload_watch.py:15-95.)"""
    from .storage import OffloadJournal, transfer

    journal = OffloadJournal(journal_path)
    status_path = Path(journal_path).parent / "OFFLOAD_WATCH_STATUS.json"
    done = 0
    last = {}
    while cycles is None or done < cycles:
        tasks, summary = offload_plan(source, destination, minimum_bytes=minimum_bytes)
        added = grow_plan(plan_path, tasks)
        moved, errors = 0, []
        rows = [json.loads(line) for line in Path(plan_path).read_text().splitlines() if line.strip()] if Path(plan_path).exists() else []
        for row in rows:
            if journal.state(row["source"])[0] == "verified":
                continue
            try:
                transfer(row["source"], row["destination"], journal)
                moved += 1
            except (OSError, ValueError, RuntimeError) as why:
                errors.append({"source": row["source"], "error": str(why)})
        last = {"state": "needs_attention" if errors else "caught_up", "new_files": added, "transferred": moved, "errors": errors, "scan": summary, "time": time.time()}
        atomic_write_json(status_path, last)
        if errors:
            break
        done += 1
        if cycles is None or done < cycles:
            sleep(sleep_seconds)
    return last
