"""Provenance: stable content identities for datasets, source trees, weights and tokenizers.

The identities are byte-compatible with the reference's (src/archlab/provenance.py:26-389), so a manifest or a hash
written by either side verifies on the other:

* canonical JSON (sorted keys, no spaces, UTF-8) is what is hashed for structured values;
* binary material is hashed as *frames*: an 8-byte big-endian length followed by the bytes (``Frames``);
* a dataset manifest is a sorted (path, size, sha256) inventory; its inventory hash covers the file rows and its
  identity hash the whole document.  ``sha256sum`` ledgers ("<digest>  <path>" lines) load as manifests without sizes;
* a source tree is named by its commit, the hash of ``git diff --binary HEAD`` and a framed hash of every untracked
  file (name, then kind-tagged content), so a dirty tree is identified without copying it anywhere.
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
MANIFEST_KIND = "dataset-content-manifest"
_HEX = frozenset("0123456789abcdef")


class ProvenanceError(ValueError):
    pass


def canonical_json_bytes(value: Any) -> bytes:
    return json.dumps(value, ensure_ascii=False, sort_keys=True, separators=(",", ":")).encode("utf-8")


def stable_json_sha256(value: Any) -> str:
    return hashlib.sha256(canonical_json_bytes(value)).hexdigest()


class Frames:
    """SHA-256 over length-prefixed parts; several digests can be fed the same frames at once."""

    def __init__(self, *seeds: bytes):
        self.digests = [hashlib.sha256(seed) for seed in (seeds or (b"",))]

    def number(self, value: int) -> "Frames":
        for d in self.digests:
            d.update(int(value).to_bytes(8, "big"))
        return self

    def part(self, payload: bytes) -> "Frames":
        self.number(len(payload))
        for d in self.digests:
            d.update(payload)
        return self

    def hex(self, which: int = 0) -> str:
        return self.digests[which].hexdigest()


def _inside(root: Path, relative: str) -> Path:
    """``root / relative`` for a manifest path, refusing absolute paths, ``..`` and anything that resolves outside."""
    rel = Path(relative)
    if rel.is_absolute() or not rel.parts or ".." in rel.parts:
        raise ProvenanceError(f"manifest path must be safe and relative: {relative!r}")
    target = (root / rel).resolve()
    if root != Path() and root not in target.parents and target != root:
        raise ProvenanceError(f"dataset file escapes root: {relative}")
    return target


@dataclass(frozen=True)
class DatasetFile:
    path: str
    size: int | None
    sha256: str

    def validate(self) -> None:
        _inside(Path(), self.path)
        problems = {"negative size": self.size is not None and self.size < 0,
                    "invalid SHA-256": len(self.sha256) != 64 or not set(self.sha256.lower()) <= _HEX}
        for what, bad in problems.items():
            if bad:
                raise ProvenanceError(f"{what} for {self.path}")


@dataclass(frozen=True)
class DatasetManifest:
    dataset: str
    revision: str
    files: tuple[DatasetFile, ...]
    schema_version: int = SCHEMA
    kind: str = MANIFEST_KIND

    def rows(self) -> list[dict]:
        return [asdict(f) for f in self.files]

    def validate(self) -> None:
        names = [f.path for f in self.files]
        refusals = (
            ("unsupported dataset manifest schema or kind", self.schema_version != SCHEMA or self.kind != MANIFEST_KIND),
            ("dataset, revision and files must not be empty", not (self.dataset and self.revision and self.files)),
            ("dataset manifest paths must be sorted and unique", names != sorted(set(names))),
        )
        for message, bad in refusals:
            if bad:
                raise ProvenanceError(message)
        for f in self.files:
            f.validate()

    @property
    def inventory_sha256(self) -> str:
        return stable_json_sha256(self.rows())

    @property
    def identity_sha256(self) -> str:
        return stable_json_sha256(self.to_dict())

    def to_dict(self) -> dict[str, Any]:
        head = {k: getattr(self, k) for k in ("schema_version", "kind", "dataset", "revision")}
        return {**head, "inventory_sha256": self.inventory_sha256, "files": self.rows()}

    @classmethod
    def from_rows(cls, dataset: str, revision: str, rows: Iterable[DatasetFile], **extra) -> "DatasetManifest":
        manifest = cls(dataset, revision, tuple(sorted(rows, key=lambda f: f.path)), **extra)
        manifest.validate()
        return manifest


def create_dataset_manifest(root, *, dataset: str, revision: str, patterns: Sequence[str] = ("**/*",)) -> DatasetManifest:
    root = Path(root).expanduser().resolve()
    if not root.is_dir():
        raise FileNotFoundError(root)
    found = {p.resolve() for pattern in patterns for p in root.glob(pattern) if p.is_file()}
    return DatasetManifest.from_rows(dataset, revision,
                                     (DatasetFile(p.relative_to(root).as_posix(), p.stat().st_size, sha256_file(p)) for p in found))


def write_dataset_manifest(path, manifest: DatasetManifest) -> None:
    manifest.validate()
    Path(path).write_text(json.dumps(manifest.to_dict(), indent=2, sort_keys=True) + "\n", encoding="utf-8")


def _from_ledger(text: str, name: str) -> DatasetManifest:
    rows = []
    for line in filter(None, (raw.strip() for raw in text.splitlines())):
        digest, _, file_name = line.partition("  ")
        rows.append(DatasetFile(file_name.lstrip("*./"), None, digest.lower()))
    return DatasetManifest.from_rows(name, "sha256sum-ledger", rows)


def load_dataset_manifest(path, *, dataset_root_name: str = "dataset") -> DatasetManifest:
    text = Path(path).read_text(encoding="utf-8")
    if not text.lstrip().startswith("{"):
        return _from_ledger(text, dataset_root_name)
    doc = json.loads(text)
    manifest = DatasetManifest.from_rows(doc["dataset"], doc["revision"], (DatasetFile(**row) for row in doc["files"]),
                                         schema_version=doc.get("schema_version", SCHEMA), kind=doc.get("kind", MANIFEST_KIND))
    if [f.path for f in manifest.files] != [row["path"] for row in doc["files"]]:
        raise ProvenanceError("dataset manifest paths must be sorted and unique")
    if doc.get("inventory_sha256", manifest.inventory_sha256) != manifest.inventory_sha256:
        raise ProvenanceError("dataset manifest inventory hash mismatch")
    return manifest


def verify_dataset_manifest(root, manifest_path, *, mode: str = "metadata", required_files: Iterable[str] | None = None) -> dict:
    """``metadata``: the exact file set (unless ``required_files`` narrows it) and every size; ``full``: also content."""
    if mode not in ("metadata", "full"):
        raise ProvenanceError("dataset verification mode must be metadata or full")
    root = Path(root).expanduser().resolve()
    manifest = load_dataset_manifest(Path(manifest_path).expanduser().resolve(), dataset_root_name=root.name)
    listed = {f.path: f for f in manifest.files}
    if required_files is None:
        on_disk = {p.relative_to(root).as_posix() for p in root.rglob("*") if p.is_file()}
        if on_disk != set(listed):
            raise ProvenanceError(f"dataset inventory mismatch: extra={sorted(on_disk - set(listed))[:5]} "
                                  f"missing={sorted(set(listed) - on_disk)[:5]}")
        wanted = sorted(listed)
    else:
        wanted = sorted(set(required_files))
        if absent := [name for name in wanted if name not in listed]:
            raise ProvenanceError("required files are absent from the dataset manifest: " + ", ".join(absent))
    seen_bytes = 0
    for name in wanted:
        target, row = _inside(root, name), listed[name]
        if not target.is_file():
            raise ProvenanceError(f"dataset file is missing: {name}")
        size = target.stat().st_size
        if row.size not in (None, size):
            raise ProvenanceError(f"dataset size mismatch for {name}: {size} != {row.size}")
        if mode == "full" and sha256_file(target) != row.sha256:
            raise ProvenanceError(f"dataset content mismatch for {name}")
        seen_bytes += size
    return {"dataset": manifest.dataset, "revision": manifest.revision, "mode": mode, "files": len(wanted), "bytes": seen_bytes,
            "identity_sha256": manifest.identity_sha256, "inventory_sha256": manifest.inventory_sha256}


class _WorkTree:
    def __init__(self, root: Path):
        self.root = root

    def git(self, *args: str) -> bytes:
        return subprocess.run(["git", "-c", f"safe.directory={self.root}", *args], cwd=self.root, check=True,
                              stdout=subprocess.PIPE).stdout

    def untracked(self) -> list[Path]:
        listing = self.git("ls-files", "--others", "--exclude-standard", "-z")
        return sorted(Path(os.fsdecode(raw)) for raw in listing.split(b"\0") if raw)

    def content(self, rel: Path) -> bytes:
        """Kind-tagged bytes of an untracked entry: a symlink's target, a file's bytes, or a bare tag for anything else."""
        p = self.root / rel
        if p.is_symlink():
            return b"symlink\0" + os.fsencode(os.readlink(p))
        return b"file\0" + p.read_bytes() if p.is_file() else b"other\0"


def source_provenance(repository) -> dict[str, Any]:
    tree = _WorkTree(Path(repository).expanduser().resolve())
    diff = tree.git("diff", "--binary", "HEAD")
    extra = tree.untracked()
    frames = Frames(b"", b"tracked-diff\0" + diff)             # [0]: untracked files alone, [1]: diff + untracked files
    for rel in extra:
        frames.part(os.fsencode(rel)).part(tree.content(rel))
    return {"source_commit": tree.git("rev-parse", "HEAD").decode().strip(),
            "source_dirty": bool(tree.git("status", "--porcelain=v1", "--untracked-files=all").strip()),
            "source_diff_sha256": hashlib.sha256(diff).hexdigest(), "source_untracked_files": [str(p) for p in extra],
            "source_untracked_sha256": frames.hex(0), "source_worktree_sha256": frames.hex(1)}


def hash_named_tensors(named_tensors: Iterable[tuple[str, torch.Tensor]], *, include_names: set[str] | None = None) -> str:
    """Names, shapes, dtypes and raw bytes in name order; bit patterns (bf16, fp8) are hashed as stored."""
    picked = {name: t for name, t in named_tensors if include_names is None or name in include_names}
    if not picked:
        raise ProvenanceError("no tensors were selected for initialization hashing")
    frames = Frames()
    for name in sorted(picked):
        t = picked[name].detach().contiguous()
        frames.part(canonical_json_bytes({"name": name, "shape": list(t.shape), "dtype": str(t.dtype)}))
        frames.part(bytes(t.view(torch.uint8).cpu().untyped_storage()) if t.numel() else b"")
    return frames.hex()


def hash_tokenizer_vocabulary(tokenizer: Any, *, padded_vocab_size: int | None = None) -> str:
    """Vocabulary size, padded size, then (id, decoded bytes) of every token."""
    size = int(tokenizer.get_vocab_size())
    if padded_vocab_size is not None and padded_vocab_size < size:
        raise ProvenanceError("padded vocabulary is smaller than the tokenizer vocabulary")
    encoder = getattr(tokenizer, "enc", None)
    token_bytes = encoder.decode_single_token_bytes if hasattr(encoder, "decode_single_token_bytes") \
        else (lambda token: tokenizer.decode([token]).encode("utf-8"))
    frames = Frames().number(size).number(padded_vocab_size or size)
    for token in range(size):
        frames.number(token).part(token_bytes(token))
    return frames.hex()
