"""Checkpoint retention for explicitly configured experiment roots: keep the newest complete save, verify it, and only
then remove older complete saves; a service outside the training processes.

    python -m archlab_b200.services.retention --config policy.json --audit DIR [--apply] [--watch --interval S]

Behaviour (the reference's sweeper: src/archlab/storage/checkpoint_retention.py:45-250):

* a *policy* lists groups; a group names ``roots`` (every ``step-<n>`` child is a candidate) and / or explicit ``paths``.
  Only directories with a ``COMPLETE.json`` are candidates; they are ordered by (step, supervised tokens) of the
  marker's cursor, never by modification time.  Unfinished saves are left alone.
* before anything older is touched, the newest candidate is *verified*: rank manifests agree with the marker (contract,
  cursor, world size, rank), all ranks list the same tensors, each tensor's chunks add up to its shape, every payload
  file has a plausible length for its element count and dtype, optimizer / RNG payloads (when the manifest lists them)
  are non-empty.  The verdict is cached per marker hash, so a finished save is read once.
* holds: a save is kept when the policy protects its path or step, or when it carries ``PINNED.json``,
  ``EVAL_PENDING.json`` or a reader lease under ``.checkpoint-readers/``.
* removal is two-phase and resumable: manifests are archived under ``<audit>/deleted/<key>/``, a receipt is written, the
  directory is renamed to ``.retention-delete-<key>`` next to it, deleted, and the receipt is completed.  A sweep that
  finds an incomplete receipt finishes exactly that staged directory and nothing else.  Symlinks anywhere in a candidate
  are refused.
* ``LATEST.json`` in every root and in the audit directory records the outcome; one sweeper per audit directory
  (``LOCK``, non-blocking).
"""
from __future__ import annotations

import argparse
import fcntl
import hashlib
import json
import math
import os
import re
import shutil
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from datetime import datetime, timezone
from pathlib import Path

from ..contracts.substrate import atomic_write_json

SHARDED_FORMAT = "archlab-v41-full-sharded-v1"
ELEMENT_BYTES = {"bfloat16": 2, "float16": 2, "float32": 4, "float64": 8, "int64": 8, "int32": 4, "int16": 2, "int8": 1, "uint8": 1,
                 "bool": 1, "float8_e4m3fn": 1, "float8_e5m2": 1}
CONTAINER_SLACK = 65536              # a serialised chunk is its raw bytes plus less than this much container overhead
HOLD_MARKERS = ("PINNED.json", "EVAL_PENDING.json")
STAGED_PREFIX = ".retention-delete-"
_STEP_DIR = re.compile(r"step-\d+")


def _now() -> str:
    return datetime.now(timezone.utc).isoformat()


def _key(path: Path) -> str:
    return hashlib.sha256(str(path).encode()).hexdigest()[:20]


def _refuse_symlinks(root: Path, target: Path) -> Path:
    """``target`` must live under ``root`` with no symlink on the way (a link could point a deletion somewhere else)."""
    if not target.resolve().is_relative_to(root.resolve()):
        raise ValueError(f"unsafe checkpoint path: {target}")
    for p in (target, *target.parents):
        if p == root:
            break
        if p.is_symlink():
            raise ValueError(f"symlink in checkpoint path: {p}")
    return target


@dataclass(frozen=True)
class Candidate:
    step: int
    tokens: int
    path: Path

    def held_by(self, policy: "Policy", group: dict) -> str | None:
        if str(self.path) in policy.protected_paths:
            return "protected path"
        if self.step in policy.protected_steps | set(group.get("protected_steps", ())):
            return "protected step"
        for marker in HOLD_MARKERS:
            if (self.path / marker).exists():
                return marker
        if any((self.path / ".checkpoint-readers").glob("*.json")):
            return "reader lease"
        return None


@dataclass
class Policy:
    groups: list[dict]
    protected_paths: set[str] = field(default_factory=set)
    protected_steps: set[int] = field(default_factory=set)

    @classmethod
    def from_json(cls, doc: dict) -> "Policy":
        return cls(list(doc["groups"]), set(doc.get("protected", {})), set(doc.get("protected_steps", [])))

    @staticmethod
    def candidates(group: dict) -> list[Candidate]:
        paths = [Path(p) for p in group.get("paths", [])]
        for root in map(Path, group.get("roots", [])):
            if root.is_symlink() or root.resolve() != root:
                raise ValueError("root must be absolute and contain no symlinks")
            paths += [p for p in root.glob("step-*") if _STEP_DIR.fullmatch(p.name)]
        found = []
        for path in paths:
            if path.is_symlink():
                raise ValueError(f"symlink candidate: {path}")
            marker = path / "COMPLETE.json"
            if marker.exists():
                cursor = json.loads(marker.read_text())["cursor"]
                found.append(Candidate(int(cursor["step"]), int(cursor.get("supervised_tokens", 0)), path))
        return sorted(found, key=lambda c: (c.step, c.tokens, str(c.path)))


def verify_sharded(path: Path) -> dict:
    """Structural verification of one full-sharded save (no tensor payload is read)."""
    if path.is_symlink():
        raise ValueError(f"symlink checkpoint: {path}")
    marker = json.loads(_refuse_symlinks(path, path / "COMPLETE.json").read_text())
    if marker["format"] != SHARDED_FORMAT:
        raise ValueError("unsupported checkpoint format")
    world = marker["world_size"]
    manifests = marker.get("manifests") or [f"rank-{r:02d}/MANIFEST.json" for r in range(world)]
    if len(manifests) != world or len(set(manifests)) != world:
        raise ValueError("missing or duplicated rank manifests")
    checked, names = 0, None
    for rank, relative in enumerate(manifests):
        manifest_path = _refuse_symlinks(path, path / relative)
        manifest = json.loads(manifest_path.read_text())
        for agreed in ("contract", "cursor", "world_size"):
            if manifest[agreed] != marker[agreed]:
                raise ValueError(f"rank {rank} {agreed} mismatch")
        if manifest["rank"] != rank:
            raise ValueError("rank mismatch")
        listed = [t["name"] for t in manifest["tensors"]]
        if names not in (None, listed):
            raise ValueError("tensor names differ across ranks")
        names = listed
        here = manifest_path.parent
        for t in manifest["tensors"]:
            if sum(c["elements"] for c in t["chunks"]) != math.prod(t["shape"]):
                raise ValueError(f"tensor chunks incomplete: {t['name']}")
            width = ELEMENT_BYTES[t["dtype"].removeprefix("torch.")]
            for chunk in t["chunks"]:
                payload = _refuse_symlinks(path, here / chunk["file"])
                raw, size = chunk["elements"] * width, payload.stat().st_size
                if not raw <= size < raw + CONTAINER_SLACK:
                    raise ValueError(f"bad payload length: {payload}")
                checked += 1
        extras = [*manifest.get("optimizer_states", []), *(["rng.pt"] if "optimizer_states" in manifest else [])]
        for name in extras:
            if _refuse_symlinks(path, here / name).stat().st_size <= 0:
                raise ValueError(f"empty payload: {here / name}")
            checked += 1
    return {"path": str(path), "cursor": marker["cursor"], "ranks": world, "payload_files_checked": checked, "validated_utc": _now(),
            "validation": "rank identities, tensor element counts and payload lengths; optimizer/RNG presence where listed"}


def _walk(path: Path) -> tuple[list[Path], int]:
    """Every file under ``path`` and their total size; refuses symlinks and special files."""
    files, pending = [], [path]
    while pending:
        with os.scandir(pending.pop()) as entries:
            for entry in entries:
                if entry.is_symlink():
                    raise ValueError(f"symlink inside deletion candidate: {entry.path}")
                if entry.is_dir(follow_symlinks=False):
                    pending.append(Path(entry.path))
                elif entry.is_file(follow_symlinks=False):
                    files.append(Path(entry.path))
                else:
                    raise ValueError(f"unexpected checkpoint entry: {entry.path}")
    with ThreadPoolExecutor(max_workers=8) as pool:                # metadata only; network file systems answer these slowly
        total = sum(pool.map(lambda p: p.stat().st_size, files))
    return files, total


def _delete(path: Path) -> None:
    def drop(child: Path):
        shutil.rmtree(child) if child.is_dir() and not child.is_symlink() else child.unlink()

    with ThreadPoolExecutor(max_workers=8) as pool:                # rank directories are independent
        list(pool.map(drop, list(path.iterdir())))
    path.rmdir()


class Sweeper:
    def __init__(self, audit: Path, *, apply: bool = False, write=atomic_write_json):
        self.audit, self.apply, self._write = Path(audit), apply, write
        self.audit.mkdir(parents=True, exist_ok=True)

    # ---- two-phase removal ---------------------------------------------------------------------------------------
    def finish_interrupted(self) -> list[str]:
        """Complete removals whose receipt says the rename happened but the deletion did not."""
        finished = []
        for file in (self.audit / "deleted").glob("*/RECEIPT.json"):
            receipt = json.loads(file.read_text())
            staged = Path(receipt["staged"])
            if receipt["complete"] or not staged.exists():
                continue
            if staged.is_symlink() or not staged.name.startswith(STAGED_PREFIX):
                raise ValueError("unsafe pending deletion")
            _delete(staged)
            self._write(file, {**receipt, "complete": True, "completed_utc": _now()})
            finished.append(str(staged))
        return finished

    def remove(self, path: Path, replacement: Path) -> dict:
        files, size = _walk(path)
        key = _key(path)
        archive = self.audit / "deleted" / key
        for source in files:
            if source.name in ("COMPLETE.json", "MANIFEST.json"):         # what the save was stays on record
                kept = archive / source.relative_to(path)
                kept.parent.mkdir(parents=True, exist_ok=True)
                shutil.copy2(source, kept)
        archive.mkdir(parents=True, exist_ok=True)
        staged = path.with_name(STAGED_PREFIX + key)
        receipt = {"original": str(path), "staged": str(staged), "replacement": str(replacement), "bytes": size,
                   "started_utc": _now(), "complete": False}
        self._write(archive / "RECEIPT.json", receipt)
        path.rename(staged)
        _delete(staged)
        receipt.update(complete=True, completed_utc=_now())
        self._write(archive / "RECEIPT.json", receipt)
        return receipt

    # ---- verification cache --------------------------------------------------------------------------------------
    def verified(self, newest: Path) -> str:
        digest = hashlib.sha256((newest / "COMPLETE.json").read_bytes()).hexdigest()
        cache = self.audit / f"verified-{_key(newest)}.json"
        if not cache.exists() or json.loads(cache.read_text()).get("marker_sha256") != digest:
            self._write(cache, {**verify_sharded(newest), "marker_sha256": digest})
        return digest

    # ---- one pass ------------------------------------------------------------------------------------------------
    def sweep_group(self, policy: Policy, group: dict) -> dict | None:
        ordered = Policy.candidates(group)
        if not ordered:
            return None
        newest = ordered[-1].path
        holds = {str(c.path): why for c in ordered[:-1] if (why := c.held_by(policy, group))}
        doomed = [c.path for c in ordered[:-1] if str(c.path) not in holds]
        digest = self.verified(newest)                               # nothing is removed unless the survivor checks out
        record = {"name": group["name"], "newest": str(newest), "delete": [str(p) for p in doomed], "held": holds}
        if self.apply:
            for root in group.get("roots", []):
                self._write(Path(root) / "LATEST.json", {"path": str(newest), "marker_sha256": digest, "utc": _now()})
            record["removed"] = [self.remove(p, newest) for p in doomed]
        return record

    def sweep(self, policy: Policy) -> dict:
        result = {"utc": _now(), "apply": self.apply, "groups": [], "errors": []}
        if self.apply:
            result["resumed"] = self.finish_interrupted()
        for group in policy.groups:
            try:
                if (record := self.sweep_group(policy, group)) is not None:
                    result["groups"].append(record)
            except Exception as error:                               # one broken group must not stop the others
                result["errors"].append({"group": group.get("name"), "error": repr(error)})
        self._write(self.audit / "LATEST.json", result)
        return result


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", type=Path, required=True)
    ap.add_argument("--audit", type=Path, required=True)
    ap.add_argument("--apply", action="store_true")
    ap.add_argument("--watch", action="store_true")
    ap.add_argument("--interval", type=float, default=60)
    a = ap.parse_args(argv)
    if not 1 <= a.interval <= 60:
        raise SystemExit("interval must be between 1 and 60 seconds")
    a.audit.mkdir(parents=True, exist_ok=True)
    with (a.audit / "LOCK").open("w") as lock:
        try:
            fcntl.flock(lock, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except BlockingIOError:
            print("retention is already running for this policy", flush=True)
            return 0
        sweeper = Sweeper(a.audit, apply=a.apply)
        while True:
            result = sweeper.sweep(Policy.from_json(json.loads(a.config.read_text())))     # the policy is re-read every pass
            print(json.dumps(result), flush=True)
            if not a.watch:
                return 1 if result["errors"] else 0
            time.sleep(a.interval)


if __name__ == "__main__":
    raise SystemExit(main())


def checkpoint_receipt(path, *, sample_tensors: tuple[str, ...] = (), sample_ranks: tuple[int, ...] = (0,)) -> dict:
    """The structural verification plus REPRESENTATIVE content checks: for the named tensors (default: the first and the
    last tensor of the manifest) the first chunk on each sampled rank is loaded and its SHA-256 compared with the
    manifest.  Reading every payload of a multi-terabyte save is the restore's job; a receipt that proves lengths
    everywhere and content somewhere is what an archive step can afford
    (src/archlab/storage/v41_checkpoint_receipt.py:13-94)."""
    import hashlib

    import torch

    path = Path(path)
    base = verify_sharded(path)
    marker = json.loads((path / "COMPLETE.json").read_text())
    manifests = marker.get("manifests") or [f"rank-{r:02d}/MANIFEST.json" for r in range(marker["world_size"])]
    samples = []
    for rank in sample_ranks:
        manifest_path = path / manifests[rank]
        tensors = json.loads(manifest_path.read_text())["tensors"]
        wanted = sample_tensors or tuple(dict.fromkeys((tensors[0]["name"], tensors[-1]["name"])))
        for name in wanted:
            entry = next((t for t in tensors if t["name"] == name), None)
            if entry is None:
                raise ValueError(f"sampled tensor is not in the checkpoint: {name}")
            chunk = entry["chunks"][0]
            value = torch.load(manifest_path.parent / chunk["file"], map_location="cpu", weights_only=True)
            digest = hashlib.sha256(value.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()
            if digest != chunk["sha256"]:
                raise ValueError(f"payload checksum mismatch: rank {rank} {name}")
            samples.append({"rank": rank, "name": name, "sha256": digest, "verified": True})
    return {**base, "passed": True, "representative_checksums": samples, "all_payload_lengths_verified": True}
