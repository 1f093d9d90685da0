"""Provenance: stable content identities for datasets, source trees, weights and tokenizers
(src/archlab/provenance.py:26-389).

* dataset manifests: sorted (path, size, sha256) inventories; ``verify`` in ``metadata`` mode checks the
  exact file set and sizes, ``full`` mode re-hashes every file; legacy ``sha256sum`` ledgers load too.
* ``source_provenance``: commit + hashes of the tracked diff and of untracked file contents, so a dirty
  work tree is identified without exposing it.
* ``hash_named_tensors``: names, shapes, dtypes and raw bytes in name order (bit patterns of bf16 /
  fp8 preserved).  ``hash_tokenizer_vocabulary``: every token's decoded bytes.
"""
from __future__ import annotations

import hashlib
import json
import os
import subprocess
from collections.abc import Iterable, Sequence
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any

import torch

from .substrate import sha256_file

SCHEMA = 1


class ProvenanceError(ValueError):
    pass


def canonical_json_bytes(value: Any) -> bytes:
    return json.dumps(value, ensure_ascii=False, sort_keys=True, separators=(",", ":")).encode("utf-8")


def stable_json_sha256(value: Any) -> str:
    return hashlib.sha256(canonical_json_bytes(value)).hexdigest()


def _safe_relative(value: str) -> Path:
    p = Path(value)
    if p.is_absolute() or not p.parts or ".." in p.parts:
        raise ProvenanceError(f"manifest path must be safe and relative: {value!r}")
    return p


@dataclass(frozen=True)
class DatasetFile:
    path: str
    size: int | None
    sha256: str

    def validate(self) -> None:
        _safe_relative(self.path)
        if self.size is not None and self.size < 0:
            raise ProvenanceError(f"negative size for {self.path}")
        if len(self.sha256) != 64 or any(c not in "0123456789abcdef" for c in self.sha256.lower()):
            raise ProvenanceError(f"invalid SHA-256 for {self.path}")


@dataclass(frozen=True)
class DatasetManifest:
    dataset: str
    revision: str
    files: tuple[DatasetFile, ...]
    schema_version: int = SCHEMA
    kind: str = "dataset-content-manifest"

    def validate(self) -> None:
        if self.schema_version != SCHEMA or self.kind != "dataset-content-manifest":
            raise ProvenanceError("unsupported dataset manifest schema or kind")
        if not self.dataset or not self.revision or not self.files:
            raise ProvenanceError("dataset, revision and files must not be empty")
        paths = [f.path for f in self.files]
        if paths != sorted(paths) or len(paths) != len(set(paths)):
            raise ProvenanceError("dataset manifest paths must be sorted and unique")
        for f in self.files:
            f.validate()

    @property
    def inventory_sha256(self) -> str:
        return stable_json_sha256([asdict(f) for f in self.files])

    @property
    def identity_sha256(self) -> str:
        return stable_json_sha256(self.to_dict())

    def to_dict(self) -> dict[str, Any]:
        return {"schema_version": self.schema_version, "kind": self.kind, "dataset": self.dataset, "revision": self.revision,
                "inventory_sha256": self.inventory_sha256, "files": [asdict(f) for f in self.files]}


def create_dataset_manifest(root, *, dataset: str, revision: str, patterns: Sequence[str] = ("**/*",)) -> DatasetManifest:
    root = Path(root).expanduser().resolve()
    if not root.is_dir():
        raise FileNotFoundError(root)
    paths = sorted({p.resolve() for pat in patterns for p in root.glob(pat) if p.is_file()})
    files = tuple(DatasetFile(p.relative_to(root).as_posix(), p.stat().st_size, sha256_file(p)) for p in paths)
    m = DatasetManifest(dataset, revision, tuple(sorted(files, key=lambda f: f.path)))
    m.validate()
    return m


def write_dataset_manifest(path, manifest: DatasetManifest) -> None:
    manifest.validate()
    Path(path).write_text(json.dumps(manifest.to_dict(), indent=2, sort_keys=True) + "\n", encoding="utf-8")


def load_dataset_manifest(path, *, dataset_root_name: str = "dataset") -> DatasetManifest:
    path = Path(path)
    text = path.read_text(encoding="utf-8")
    if text.lstrip().startswith("{"):
        d = json.loads(text)
        m = DatasetManifest(d["dataset"], d["revision"], tuple(DatasetFile(**f) for f in d["files"]),
                            d.get("schema_version", SCHEMA), d.get("kind", "dataset-content-manifest"))
        if "inventory_sha256" in d and d["inventory_sha256"] != m.inventory_sha256:
            raise ProvenanceError("dataset manifest inventory hash mismatch")
    else:                                                # legacy `sha256sum` ledger: "<hash>  <path>" lines
        files = []
        for line in text.splitlines():
            if line.strip():
                digest, _, name = line.strip().partition("  ")
                files.append(DatasetFile(name.lstrip("*./"), None, digest.lower()))
        m = DatasetManifest(dataset_root_name, "sha256sum-ledger", tuple(sorted(files, key=lambda f: f.path)))
    m.validate()
    return m


def verify_dataset_manifest(root, manifest_path, *, mode: str = "metadata", required_files: Iterable[str] | None = None) -> dict:
    if mode not in ("metadata", "full"):
        raise ProvenanceError("dataset verification mode must be metadata or full")
    root = Path(root).expanduser().resolve()
    manifest = load_dataset_manifest(Path(manifest_path).expanduser().resolve(), dataset_root_name=root.name)
    expected = {f.path: f for f in manifest.files}
    selected = sorted(set(expected) if required_files is None else set(required_files))
    if unknown := set(selected) - set(expected):
        raise ProvenanceError("required files are absent from the dataset manifest: " + ", ".join(sorted(unknown)))
    if required_files is None:
        visible = {p.relative_to(root).as_posix() for p in root.rglob("*") if p.is_file()}
        extras, missing = visible - set(expected), set(expected) - visible
        if extras or missing:
            raise ProvenanceError(f"dataset inventory mismatch: extra={sorted(extras)[:5]} missing={sorted(missing)[:5]}")
    total = 0
    for rel in selected:
        item = expected[rel]
        p = (root / _safe_relative(rel)).resolve()
        try:
            p.relative_to(root)
        except ValueError as e:
            raise ProvenanceError(f"dataset file escapes root: {rel}") from e
        if not p.is_file():
            raise ProvenanceError(f"dataset file is missing: {rel}")
        size = p.stat().st_size
        total += size
        if item.size is not None and size != item.size:
            raise ProvenanceError(f"dataset size mismatch for {rel}: {size} != {item.size}")
        if mode == "full" and sha256_file(p) != item.sha256:
            raise ProvenanceError(f"dataset content mismatch for {rel}")
    return {"dataset": manifest.dataset, "revision": manifest.revision, "mode": mode, "files": len(selected),
            "bytes": total, "identity_sha256": manifest.identity_sha256, "inventory_sha256": manifest.inventory_sha256}


def _git(root: Path, *args: str) -> bytes:
    return subprocess.run(["git", "-c", f"safe.directory={root}", *args], cwd=root, check=True, stdout=subprocess.PIPE).stdout


def source_provenance(repository) -> dict[str, Any]:
    root = Path(repository).expanduser().resolve()
    status = _git(root, "status", "--porcelain=v1", "--untracked-files=all").decode()
    diff = _git(root, "diff", "--binary", "HEAD")
    untracked = sorted(Path(os.fsdecode(p)) for p in _git(root, "ls-files", "--others", "--exclude-standard", "-z").split(b"\0") if p)
    u_digest, w_digest = hashlib.sha256(), hashlib.sha256(b"tracked-diff\0" + diff)
    for rel in untracked:
        p = root / rel
        content = (b"symlink\0" + os.fsencode(os.readlink(p))) if p.is_symlink() else \
            (b"file\0" + p.read_bytes()) if p.is_file() else b"other\0"
        name = os.fsencode(rel)
        framed = len(name).to_bytes(8, "big") + name + len(content).to_bytes(8, "big") + content
        u_digest.update(framed)
        w_digest.update(framed)
    return {"source_commit": _git(root, "rev-parse", "HEAD").decode().strip(), "source_dirty": bool(status.strip()),
            "source_diff_sha256": hashlib.sha256(diff).hexdigest(), "source_untracked_files": [str(p) for p in untracked],
            "source_untracked_sha256": u_digest.hexdigest(), "source_worktree_sha256": w_digest.hexdigest()}


def hash_named_tensors(named_tensors: Iterable[tuple[str, torch.Tensor]], *, include_names: set[str] | None = None) -> str:
    digest = hashlib.sha256()
    chosen = sorted(((n, t) for n, t in named_tensors if include_names is None or n in include_names), key=lambda kv: kv[0])
    if not chosen:
        raise ProvenanceError("no tensors were selected for initialization hashing")
    for name, t in chosen:
        d = t.detach().contiguous()
        header = canonical_json_bytes({"name": name, "shape": list(d.shape), "dtype": str(d.dtype)})
        payload = bytes(d.view(torch.uint8).cpu().untyped_storage()) if d.numel() else b""
        for part in (header, payload):
            digest.update(len(part).to_bytes(8, "big"))
            digest.update(part)
    return digest.hexdigest()


def hash_tokenizer_vocabulary(tokenizer: Any, *, padded_vocab_size: int | None = None) -> str:
    n = int(tokenizer.get_vocab_size())
    if padded_vocab_size is not None and padded_vocab_size < n:
        raise ProvenanceError("padded vocabulary is smaller than the tokenizer vocabulary")
    digest = hashlib.sha256()
    digest.update(n.to_bytes(8, "big"))
    digest.update((padded_vocab_size or n).to_bytes(8, "big"))
    enc = getattr(tokenizer, "enc", None)
    for tid in range(n):
        payload = enc.decode_single_token_bytes(tid) if enc is not None and hasattr(enc, "decode_single_token_bytes") \
            else tokenizer.decode([tid]).encode("utf-8")
        digest.update(tid.to_bytes(8, "big"))
        digest.update(len(payload).to_bytes(8, "big"))
        digest.update(payload)
    return digest.hexdigest()
