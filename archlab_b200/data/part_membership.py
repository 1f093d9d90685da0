"""One strict membership check for every trainer that reads an indexed-data tree.

A tree has ``train/part-*.bin`` and ``val/part-*.bin`` with an ``.idx`` and a ``.json`` beside every ``.bin``, and a
``DATA_READY.json`` whose ``train_parts`` / ``valid_parts`` name the part prefixes (relative to the tree or absolute).
``validated_data_prefixes`` returns the prefixes only if the files on disk are EXACTLY the declared ones: a part that
was added, removed or left empty after the manifest was sealed changes what a resumed run would read, so any
difference is an error that names the missing and the undeclared parts.
(Reference: src/archlab/megatron/indexed_data.py:9-56.)
"""
from __future__ import annotations

import json
from pathlib import Path

SUFFIXES = (".bin", ".idx", ".json")


def data_prefixes(data_root, split: str) -> list[Path]:
    data_root = Path(data_root)
    prefixes = sorted(p.with_suffix("") for p in (data_root / split).glob("part-*.bin"))
    if not prefixes:
        raise FileNotFoundError(f"no {split} part-*.bin files under {data_root}")
    for prefix in prefixes:
        for suffix in SUFFIXES:
            artifact = Path(f"{prefix}{suffix}")
            if not artifact.is_file() or artifact.stat().st_size <= 0:
                raise FileNotFoundError(f"missing or empty indexed-data artifact: {artifact}")
    return prefixes


def _declared(root: Path, ready: dict, key: str) -> set[Path]:
    names = ready.get(key)
    if not isinstance(names, list) or not names or not all(isinstance(n, str) and n for n in names):
        raise RuntimeError(f"the indexed-data manifest lacks a valid non-empty {key}")
    resolved = [(Path(n).expanduser() if Path(n).expanduser().is_absolute() else root / n).resolve() for n in names]
    if len(set(resolved)) != len(resolved):
        raise RuntimeError(f"the indexed-data manifest has duplicate {key}")
    return set(resolved)


def sealed_parts(data_root) -> dict[str, list[Path]]:
    """``{"train": [...], "val": [...]}`` part prefixes, or an error that names what differs from ``DATA_READY.json``."""
    root = Path(data_root).expanduser().resolve()
    manifest = root / "DATA_READY.json"
    try:
        ready = json.loads(manifest.read_text())
    except (OSError, json.JSONDecodeError) as why:
        raise RuntimeError(f"invalid indexed-data manifest: {manifest}") from why
    if not isinstance(ready, dict):
        raise RuntimeError(f"the indexed-data manifest must hold an object: {manifest}")
    parts = {}
    for split, key in (("train", "train_parts"), ("val", "valid_parts")):
        declared = _declared(root, ready, key)
        on_disk = [p.resolve() for p in data_prefixes(root, split)]
        if declared != set(on_disk):
            missing, extra = sorted(map(str, declared - set(on_disk))), sorted(map(str, set(on_disk) - declared))
            raise RuntimeError(f"indexed-data membership changed for {split}: missing={missing}, undeclared={extra}")
        parts[split] = on_disk
    return parts


def validated_data_prefixes(data_root) -> tuple[list[Path], list[Path]]:
    parts = sealed_parts(data_root)
    return parts["train"], parts["val"]
