"""Task-parallel corpus tokenisation with per-part READY markers, resumption and verified reuse of earlier versions.

A *contract* (``manifest.json``) freezes what is being prepared: the tokenizer identity, the rendering rules, the split
rule and the list of *tasks* (a source file and a row range each).  Any number of workers call ``run_task`` for the tasks
they are given; each task renders and tokenises its rows into a scratch directory, writes

    <partition>.bin   int32 token ids of all documents of the partition, back to back
    <partition>.idx   int64 document end offsets
    <partition>.metadata.jsonl.gz   one line per document (source row, token count, flags)

for every partition (train / heldout, decided per document group by a stable hash), then ``READY.json`` with the
inventory (sizes and SHA-256 of every file, document and token counts, the task's and the contract's hashes) and
finally publishes the directory with one rename.  A task whose published part verifies is skipped on re-runs; a part
of an *earlier dataset version* may be adopted instead of recomputed when the earlier contract differs from the current
one only in keys the caller declares harmless (``reuse_parts``): payloads are copied, re-verified and re-marked with
their origin.  ``finalise`` writes ``COMPLETE.json`` once every task has a verified part.

The reference prepares its math / agentic corpora this way (src/archlab/preprocessing/nemotron_math.py:1-621,
reuse.py:52-113); renderers and filters are supplied by the caller here.
"""
from __future__ import annotations

import gzip
import hashlib
import json
import os
import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Iterable

import numpy as np

from .prepare import split_by_group

FORMAT = "archlab-prepared-corpus-v1"
SUFFIXES = (".bin", ".idx", ".metadata.jsonl.gz")


def json_sha256(value) -> str:
    return hashlib.sha256(json.dumps(value, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def file_sha256(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _write_json(path: Path, value) -> None:
    tmp = path.with_name(f".{path.name}.tmp")
    tmp.write_text(json.dumps(value, indent=1, sort_keys=True) + "\n")
    os.replace(tmp, path)


@dataclass(frozen=True)
class Contract:
    """The frozen description of one dataset version."""
    body: dict

    @classmethod
    def create(cls, root, *, tokenizer_sha256: str, renderer_sha256: str, tasks: list[dict], heldout_fraction: float = 0.0,
               split_seed: int = 0, extra: dict | None = None) -> "Contract":
        ids = [t["id"] for t in tasks]
        if len(ids) != len(set(ids)) or any(t["rows"] <= 0 or t["row_start"] < 0 for t in tasks):
            raise ValueError("tasks need unique ids and positive row ranges")
        body = {"format": FORMAT, "tokenizer_sha256": tokenizer_sha256, "renderer_sha256": renderer_sha256, "tasks": tasks,
                "heldout_fraction": heldout_fraction, "split_seed": split_seed, **(extra or {})}
        root = Path(root)
        root.mkdir(parents=True, exist_ok=True)
        existing = root / "manifest.json"
        if existing.exists():
            if json.loads(existing.read_text()) != body:
                raise ValueError("the directory holds a different dataset contract")
        else:
            _write_json(existing, body)
        return cls(body)

    @classmethod
    def load(cls, root) -> "Contract":
        body = json.loads((Path(root) / "manifest.json").read_text())
        if body.get("format") != FORMAT:
            raise ValueError("not a prepared corpus of this framework")
        return cls(body)

    @property
    def sha256(self) -> str:
        return json_sha256(self.body)

    def task(self, task_id: str) -> dict:
        return next(t for t in self.body["tasks"] if t["id"] == task_id)


def verify_part(directory, *, task: dict | None = None, contract_sha256: str | None = None) -> dict:
    """Checks a part against its own READY marker (inventory, sizes, hashes, counts) and, when given, against the task
    and the contract it claims to belong to."""
    directory = Path(directory)
    ready = json.loads((directory / "READY.json").read_text())
    expected = {summary["prefix"] + s for summary in ready["partitions"].values() for s in SUFFIXES}
    names = [f["name"] for f in ready["files"]]
    if len(names) != len(set(names)) or set(names) != expected or any(Path(n).name != n for n in names):
        raise ValueError("part inventory is invalid")
    for f in ready["files"]:
        path = directory / f["name"]
        if path.stat().st_size != f["bytes"] or file_sha256(path) != f["sha256"]:
            raise ValueError(f"part payload changed: {f['name']}")
    if (sum(p["documents"] for p in ready["partitions"].values()) != ready["documents"]
            or sum(p["tokens"] for p in ready["partitions"].values()) != ready["tokens"]):
        raise ValueError("part counts do not add up")
    if task is not None:
        covered = ready["documents"] + ready.get("excluded_documents", 0)
        if ready["id"] != task["id"] or ready["task_sha256"] != json_sha256(task) or covered != task["rows"]:
            raise ValueError("part does not cover its task")
    if contract_sha256 is not None and ready["contract_sha256"] != contract_sha256:
        raise ValueError("part belongs to another contract")
    return ready


def _publish(scratch: Path, destination: Path) -> None:
    destination.parent.mkdir(parents=True, exist_ok=True)
    if destination.exists():
        raise FileExistsError(f"{destination} was published meanwhile")
    os.replace(scratch, destination)                       # one rename: readers see no part or the whole part


def run_task(root, task_id: str, rows: Iterable[dict], render: Callable[[dict], str | None], tokenizer, *, eod: int,
             group_of: Callable[[dict], str] = lambda row: str(row.get("id", "")), scratch=None,
             meta_of: Callable[[dict], dict] | None = None) -> dict:
    """Prepares one task.  ``rows`` yields exactly the task's row range; ``render`` returns the document text or None to
    exclude the row (excluded rows are counted, so coverage stays checkable).  ``meta_of(row)`` adds fields to the
    document's metadata line (a problem hash for later overlap audits, a source id)."""
    root = Path(root)
    contract = Contract.load(root)
    task = contract.task(task_id)
    destination = root / "parts" / task_id
    if destination.exists():
        return verify_part(destination, task=task, contract_sha256=contract.sha256)         # done earlier: skip
    work = Path(scratch or root / ".scratch") / f"{task_id}.{os.getpid()}"
    shutil.rmtree(work, ignore_errors=True)
    work.mkdir(parents=True)
    parts = {name: {"tokens": [], "ends": [], "meta": []} for name in ("train", "heldout")}
    excluded, seen = 0, 0
    for offset, row in enumerate(rows):
        seen += 1
        text = render(row)
        if text is None:
            excluded += 1
            continue
        ids = list(tokenizer.encode(text)) + [eod]
        side = "heldout" if split_by_group(group_of(row), contract.body["split_seed"], contract.body["heldout_fraction"]) else "train"
        p = parts[side]
        p["tokens"].extend(ids)
        p["ends"].append(len(p["tokens"]))
        p["meta"].append({**(meta_of(row) if meta_of else {}), "row": task["row_start"] + offset, "tokens": len(ids)})
    if seen != task["rows"]:
        shutil.rmtree(work, ignore_errors=True)
        raise ValueError(f"task {task_id} expected {task['rows']} rows, the source gave {seen}")
    files, summaries = [], {}
    for name, p in parts.items():
        prefix = f"{task_id}-{name}"
        np.asarray(p["tokens"], dtype=np.int32).tofile(work / (prefix + ".bin"))
        np.asarray(p["ends"], dtype=np.int64).tofile(work / (prefix + ".idx"))
        with gzip.open(work / (prefix + ".metadata.jsonl.gz"), "wt") as f:
            f.writelines(json.dumps(m) + "\n" for m in p["meta"])
        summaries[name] = {"prefix": prefix, "documents": len(p["ends"]), "tokens": len(p["tokens"])}
        files += [{"name": prefix + s, "bytes": (work / (prefix + s)).stat().st_size, "sha256": file_sha256(work / (prefix + s))} for s in SUFFIXES]
    ready = {"id": task_id, "task_sha256": json_sha256(task), "contract_sha256": contract.sha256, "source": task.get("source"),
             "row_start": task["row_start"], "documents": sum(s["documents"] for s in summaries.values()),
             "tokens": sum(s["tokens"] for s in summaries.values()), "excluded_documents": excluded, "partitions": summaries, "files": files}
    _write_json(work / "READY.json", ready)
    verify_part(work, task=task, contract_sha256=contract.sha256)
    _publish(work, destination)
    return ready


def reuse_parts(root, earlier_root, *, harmless_keys: set[str]) -> dict:
    """Adopts verified parts of an earlier dataset version for tasks that are identical in both contracts.  The two
    contracts may differ only in ``harmless_keys`` (plus the task lists themselves, compared task by task); payloads are
    copied, not linked, and re-verified after the copy."""
    root, earlier_root = Path(root), Path(earlier_root).resolve()
    current, earlier = Contract.load(root), Contract.load(earlier_root)
    ignore = set(harmless_keys) | {"tasks"}
    if {k: v for k, v in current.body.items() if k not in ignore} != {k: v for k, v in earlier.body.items() if k not in ignore}:
        raise ValueError("the earlier contract differs in more than the declared keys")
    adopted, skipped = [], []
    for task in current.body["tasks"]:
        source, destination = earlier_root / "parts" / task["id"], root / "parts" / task["id"]
        if destination.exists() or not (source / "READY.json").exists():
            continue
        try:
            origin = verify_part(source, contract_sha256=earlier.sha256)
            if origin["task_sha256"] != json_sha256(task):
                raise ValueError("task changed between the versions")
        except (ValueError, KeyError, FileNotFoundError) as why:
            skipped.append({"id": task["id"], "reason": str(why)})
            continue
        work = root / ".scratch" / f"{task['id']}.reuse.{os.getpid()}"
        shutil.rmtree(work, ignore_errors=True)
        work.mkdir(parents=True)
        for f in origin["files"]:
            shutil.copyfile(source / f["name"], work / f["name"])
        _write_json(work / "ORIGIN_READY.json", origin)
        _write_json(work / "READY.json", {**origin, "contract_sha256": current.sha256,
                                          "reused_from": {"directory": str(source), "contract_sha256": earlier.sha256,
                                                          "ready_sha256": file_sha256(source / "READY.json")}})
        verify_part(work, task=task, contract_sha256=current.sha256)
        _publish(work, destination)
        adopted.append(task["id"])
    return {"adopted": adopted, "skipped": skipped}


def finalise(root) -> dict:
    """``COMPLETE.json`` once every task has a verified part; names what is missing otherwise."""
    root = Path(root)
    contract = Contract.load(root)
    missing = [t["id"] for t in contract.body["tasks"] if not (root / "parts" / t["id"] / "READY.json").exists()]
    if missing:
        raise ValueError("tasks without a part: " + ", ".join(missing[:10]))
    totals = {"train": {"documents": 0, "tokens": 0}, "heldout": {"documents": 0, "tokens": 0}}
    parts, excluded = {}, 0
    for t in contract.body["tasks"]:
        ready = verify_part(root / "parts" / t["id"], task=t, contract_sha256=contract.sha256)
        parts[t["id"]] = file_sha256(root / "parts" / t["id"] / "READY.json")
        excluded += ready.get("excluded_documents", 0)
        for name, s in ready["partitions"].items():
            totals[name]["documents"] += s["documents"]
            totals[name]["tokens"] += s["tokens"]
    done = {"format": FORMAT, "contract_sha256": contract.sha256, "parts": parts, "partitions": totals, "excluded_documents": excluded}
    _write_json(root / "COMPLETE.json", done)
    return done


def read_partition(root, task_id: str, partition: str) -> list[np.ndarray]:
    """Documents of one partition of one part, as int32 arrays (each ends with the end-of-document id)."""
    directory = Path(root) / "parts" / task_id
    ready = json.loads((directory / "READY.json").read_text())
    prefix = ready["partitions"][partition]["prefix"]
    tokens = np.fromfile(directory / (prefix + ".bin"), dtype=np.int32)
    ends = np.fromfile(directory / (prefix + ".idx"), dtype=np.int64)
    return [tokens[a:b] for a, b in zip([0, *ends[:-1]], ends)]
