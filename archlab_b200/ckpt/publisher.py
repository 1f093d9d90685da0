"""Starting from a model publisher's released checkpoint: the local copy is bound to a pinned manifest, byte for byte,
before any run may initialise from it.  No weight is converted or opened.

The manifest (prepared once from the publisher's immutable metadata) names the model, a 40-hex revision and, per asset,
``{bytes, sha256[, target]}``.  ``verify_publisher_checkpoint`` re-hashes every listed file NOW rather than trusting an
earlier readiness receipt; requires the assets a native load needs (configuration, generation configuration, tokenizer
files, chat template, weight index); requires the manifest to cover every shard the weight index refers to; allows a
symlinked asset only to the recorded target (shared weight stores); and refuses a directory that already holds
experiment state (an export receipt, a completion marker, RL state): an initialisation source must be pristine.
(Reference: src/archlab/training/publisher.py:12-50.)
"""
from __future__ import annotations

import json
import re
from pathlib import Path

from ..contracts.substrate import sha256_file

REQUIRED_ASSETS = frozenset({"config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "chat_template.jinja",
                             "model.safetensors.index.json"})
EXPERIMENT_STATE = ("EXPORT.json", "COMPLETE.json", "rl_state.pt")
_HEX40, _HEX64 = re.compile(r"[0-9a-f]{40}"), re.compile(r"[0-9a-f]{64}")


def build_manifest(root, *, model_id: str, revision: str) -> dict:
    """The manifest of a directory as it is now (for preparing a pin from a verified download)."""
    root = Path(root).resolve()
    assets = {}
    for path in sorted(p for p in root.iterdir() if p.is_file()):
        entry = {"bytes": path.stat().st_size, "sha256": sha256_file(path)}
        if path.is_symlink():
            entry["target"] = str(path.resolve())
        assets[path.name] = entry
    return {"schema_version": 1, "model_id": model_id, "publisher_revision": revision, "assets": assets}


def verify_publisher_checkpoint(root, manifest, *, model_id: str) -> dict:
    root, manifest = Path(root).resolve(), Path(manifest).resolve()
    record = json.loads(manifest.read_text())
    if record.get("schema_version") != 1 or record.get("model_id") != model_id or not _HEX40.fullmatch(record.get("publisher_revision", "")):
        raise ValueError("a native checkpoint needs a pinned publisher manifest")
    assets = record.get("assets", {})
    if not REQUIRED_ASSETS <= assets.keys():
        raise ValueError("the publisher manifest is missing native model / tokenizer assets")
    for name, expected in assets.items():
        if Path(name).name != name or name in (".", "..") or not _HEX64.fullmatch(expected.get("sha256", "")):
            raise ValueError("invalid publisher artifact name or hash")
        path = root / name
        if path.is_symlink() and path.resolve() != Path(expected.get("target", "")).resolve():
            raise ValueError(f"publisher artifact symlink target changed: {name}")
        if not path.is_file() or path.stat().st_size != expected.get("bytes") or sha256_file(path) != expected["sha256"]:
            raise ValueError(f"publisher artifact bytes changed: {name}")
    shards = set(json.loads((root / "model.safetensors.index.json").read_text()).get("weight_map", {}).values())
    if not shards or not shards <= assets.keys():
        raise ValueError("the publisher manifest does not cover every weight shard")
    if any(Path(s).name != s or not s.endswith(".safetensors") for s in shards):
        raise ValueError("invalid publisher weight shard")
    if any((root / name).exists() for name in EXPERIMENT_STATE):
        raise ValueError("a native publisher initialisation cannot contain experiment state")
    return {"path": str(root), "model_id": model_id, "revision": record["publisher_revision"], "manifest": str(manifest),
            "manifest_sha256": sha256_file(manifest), "files": {n: a["sha256"] for n, a in assets.items()}, "shards": len(shards),
            "initialization": "native publisher weights; fresh training state"}
