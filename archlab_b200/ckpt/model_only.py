"""Turning an older training checkpoint into a model-only evaluation checkpoint without rewriting a single weight byte.

A ``torch_dist`` iteration directory holds model tensors, optimizer moments and RNG state behind one metadata file that
maps every key to (file, offset, length).  ``export_model_only`` builds, beside the source, a staging directory in
which

* every payload file that holds at least one MODEL extent is a HARD LINK to the original (also "mixed" files that hold
  optimizer extents too: nothing is re-serialised, the weights keep their exact bytes);
* ``.metadata`` lists the model keys only (``embedding.`` / ``decoder.`` / ``output_layer.``, optionally under
  ``module.``), so a loader cannot even ask for optimizer or RNG state;
* ``EVAL_ONLY.json`` says what was dropped, how to load (no optimizer, no RNG) and that the result cannot resume training.

Before anything is published the staged checkpoint is read back through the normal distributed-checkpoint reader and
compared tensor by tensor, bit for bit, with a read of the source; every linked file must reach the last extent it is
asked for.  The latest iteration (by the tracker file), protected iterations, already converted directories and
checkpoints that another process is converting are refused.  Only with ``retire=True`` is the source moved aside and,
after the published copy verified again, deleted; the audit directory keeps the original metadata and the receipt.
(Reference: src/archlab/storage/miles_eval_checkpoint.py:379-511.)
"""
from __future__ import annotations

import copy
import fcntl
import hashlib
import json
import os
import pickle
import shutil
import time
from pathlib import Path

import torch

from ..contracts.substrate import atomic_write_json, sha256_file

FORMAT = "archlab-model-only-dcp-v1"
MODEL_PREFIXES = ("embedding.", "decoder.", "output_layer.")


def is_model_key(key: str) -> bool:
    return key.removeprefix("module.").startswith(MODEL_PREFIXES)


def _read_metadata(directory: Path):
    import torch.distributed.checkpoint as dcp

    return dcp.FileSystemReader(str(directory)).read_metadata()


def _load(directory: Path, metadata, keys) -> dict[str, torch.Tensor]:
    import torch.distributed.checkpoint as dcp

    state = {k: torch.empty(metadata.state_dict_metadata[k].size, dtype=metadata.state_dict_metadata[k].properties.dtype) for k in keys}
    dcp.load(state, checkpoint_id=str(directory))
    return state


def _same_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.dtype == b.dtype and a.shape == b.shape and torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def export_model_only(source, audit, *, retire: bool = False, protected_iterations=()) -> dict:
    source, audit = Path(source).absolute(), Path(audit).absolute()
    identity = hashlib.sha256(str(source).encode()).hexdigest()[:16]
    audit = audit / identity
    audit.mkdir(parents=True, exist_ok=True)
    with (audit / ".conversion.lock").open("a") as lock:
        try:
            fcntl.flock(lock, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except BlockingIOError as busy:
            raise ValueError("this checkpoint is already being converted") from busy
        receipt_path = audit / "receipt.json"
        if receipt_path.exists():
            receipt = json.loads(receipt_path.read_text())
            if receipt["source"] != str(source):
                raise ValueError("conversion journal identity mismatch")
            if receipt.get("phase") in ("validated", "complete"):
                return _retire(receipt, audit) if retire and receipt["phase"] == "validated" else receipt
            stale = Path(receipt["stage"])
            if stale.exists():
                shutil.rmtree(stale)
        return _convert(source, audit, identity, retire, tuple(protected_iterations))


def _convert(source: Path, audit: Path, identity: str, retire: bool, protected: tuple) -> dict:
    if source.is_symlink() or not source.is_dir() or (source / "EVAL_ONLY.json").exists():
        raise ValueError("the source must be an unconverted checkpoint directory")
    if not source.name.startswith("iter_"):
        raise ValueError("the source must be an iteration checkpoint")
    iteration = int(source.name.removeprefix("iter_"))
    if iteration in protected:
        raise ValueError("refusing to convert an explicitly protected checkpoint")
    tracker = (source.parent / "latest_checkpointed_iteration.txt").read_bytes()
    if tracker.strip() == str(iteration).encode():
        raise ValueError("refusing to convert the latest checkpoint")
    stage = source.parent / f".eval-export-{source.name}-{identity}"
    atomic_write_json(audit / "receipt.json", {"source": str(source), "stage": str(stage), "phase": "staging"})
    stage.mkdir(exist_ok=False)
    metadata = _read_metadata(source)
    models = sorted(k for k in metadata.state_dict_metadata if is_model_key(k))
    dropped = sorted(k for k in metadata.state_dict_metadata if not is_model_key(k))
    if not models:
        raise ValueError("no model tensors in the checkpoint")
    if not any(k.startswith("optimizer.") for k in dropped):
        raise ValueError("no optimizer state found in the conversion source")
    extents: dict[str, int] = {}                                    # payload file -> last byte a model extent needs
    for index, info in metadata.storage_data.items():
        if index.fqn in models:
            extents[info.relative_path] = max(extents.get(info.relative_path, 0), info.offset + info.length)
    shutil.copy2(source / ".metadata", audit / "original.metadata")
    manifest = []
    for name, end in sorted(extents.items()):
        original = source / name
        if Path(name).name != name or original.is_symlink() or not original.is_file():
            raise ValueError(f"unsafe payload file: {name}")
        os.link(original, stage / name)
        size = (stage / name).stat().st_size
        if size < end:
            raise ValueError(f"truncated model shard: {name}")
        manifest.append({"file": name, "size": size, "inode": (stage / name).stat().st_ino, "last_model_byte": end})
    exported = copy.copy(metadata)
    exported.state_dict_metadata = {k: v for k, v in metadata.state_dict_metadata.items() if k in models}
    exported.storage_data = {i: v for i, v in metadata.storage_data.items() if i.fqn in models}
    if getattr(metadata, "planner_data", None) is not None:
        exported.planner_data = {k: v for k, v in metadata.planner_data.items() if k in models}
    with (stage / ".metadata").open("wb") as f:
        pickle.dump(exported, f)
        f.flush()
        os.fsync(f.fileno())
    if (source / "common.pt").is_file():
        common = torch.load(source / "common.pt", map_location="cpu", weights_only=False)
        torch.save({k: v for k, v in common.items() if not str(k).startswith(("optimizer", "rng"))}, stage / "common.pt")
    staged, original = _load(stage, _read_metadata(stage), models), _load(source, metadata, models)
    different = [k for k in models if not _same_bits(staged[k], original[k])]
    if different:
        raise ValueError(f"staged tensors differ from the source: {different[:3]}")
    source_bytes = sum(p.stat().st_size for p in source.rglob("*") if p.is_file())
    payload = sum(row["size"] for row in manifest)
    receipt = {"format": FORMAT, "can_resume": False, "created": time.time(), "source": str(source), "stage": str(stage), "iteration": iteration,
               "source_metadata_sha256": sha256_file(source / ".metadata"), "eval_metadata_sha256": sha256_file(stage / ".metadata"),
               "model_tensors": len(models), "dropped_keys": len(dropped), "source_bytes": source_bytes, "model_payload_bytes": payload,
               "files": manifest, "validation": {"tensors_compared_bitwise": len(models)}, "load_flags": ["no optimizer", "no rng"],
               "eval_root": str(source.parent.parent / "eval-checkpoints" / source.name), "retired": False, "phase": "validated",
               "protected_iterations": list(protected), "latest_tracker_sha256": hashlib.sha256(tracker).hexdigest()}
    atomic_write_json(stage / "EVAL_ONLY.json", receipt)
    atomic_write_json(audit / "receipt.json", receipt)
    return _retire(receipt, audit) if retire else receipt


def _retire(receipt: dict, audit: Path) -> dict:
    """Publish the staged checkpoint under ``eval-checkpoints/`` and delete the source; the source is deleted last."""
    source, stage, target = Path(receipt["source"]), Path(receipt["stage"]), Path(receipt["eval_root"])
    tracker = (source.parent / "latest_checkpointed_iteration.txt").read_bytes()
    if tracker.strip() == str(receipt["iteration"]).encode():
        raise ValueError("the checkpoint became the latest one; not retiring it")
    if stage.exists():
        if target.exists():
            raise FileExistsError(f"an evaluation checkpoint already exists: {target}")
        target.parent.mkdir(parents=True, exist_ok=True)
        os.replace(stage, target)
    metadata = _read_metadata(target)
    if sha256_file(target / ".metadata") != receipt["eval_metadata_sha256"] or len(metadata.state_dict_metadata) != receipt["model_tensors"]:
        raise ValueError("the published evaluation checkpoint changed")
    _load(target, metadata, list(metadata.state_dict_metadata)[:8])          # a last read through the normal reader
    if source.exists():
        retired = source.parent / f".eval-retired-{source.name}"
        os.replace(source, retired)
        shutil.rmtree(retired)
    receipt = {**receipt, "retired": True, "phase": "complete", "stage": str(target), "completed": time.time()}
    atomic_write_json(target / "EVAL_ONLY.json", receipt)
    atomic_write_json(audit / "receipt.json", receipt)
    return receipt
