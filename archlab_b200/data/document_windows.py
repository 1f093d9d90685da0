"""Fixed-length training windows that never cross a document boundary, drawn from a weighted mixture of checksum-pinned
corpora, with train / held-out sets separated by stable document groups.

A corpus is a directory with ``manifest.json`` (format ``archlab-document-windows-v1``) naming three files by relative
path and SHA-256: ``tokens`` (1-D int32/int64 ``.npy``), ``offsets`` (document boundaries, ``offsets[0] == 0``,
``offsets[-1] == len(tokens)``, strictly increasing) and ``groups`` (a JSON list with one stable group id per document:
all documents of a task / source file share one), plus the tokenizer's file hashes.  ``write_corpus`` produces it.

``MixtureWindows`` loads every source memory-mapped after verifying format, tokenizer identity, checksums, confinement
of the asset paths, partition validity and the id range; documents shorter than a window are excluded (never padded or
joined) and counted in the receipt; each source needs eligible documents on both sides of the split.  ``sample`` picks a
source by weight, then an eligible document, then a start uniformly: the same generator state, world size and contract
give the same stream for every arm of a comparison.  Repeats are possible and count as processed, not unique, tokens.
(Reference: src/archlab/training/latent_match.py:143-213.)
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..contracts.substrate import atomic_write_json, sha256_file

FORMAT = "archlab-document-windows-v1"


@dataclass(frozen=True)
class Source:
    manifest: str
    weight: float = 1.0

    def __post_init__(self):
        if not self.manifest or not np.isfinite(self.weight) or self.weight <= 0:
            raise ValueError("each source needs a manifest and a positive finite weight")


def heldout_group(group: str, seed: int, fraction: float) -> bool:
    value = int.from_bytes(hashlib.sha256(f"document-windows:{seed}:{group}".encode()).digest()[:8], "big")
    return value < fraction * 2 ** 64


def write_corpus(directory, documents: list[np.ndarray], groups: list[str], tokenizer_files: dict[str, str]) -> Path:
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=False)
    if len(documents) != len(groups) or not documents or any(len(d) == 0 for d in documents):
        raise ValueError("one group per non-empty document")
    tokens = np.concatenate(documents).astype(np.int32)
    offsets = np.concatenate(([0], np.cumsum([len(d) for d in documents]))).astype(np.int64)
    np.save(directory / "tokens.npy", tokens)
    np.save(directory / "offsets.npy", offsets)
    (directory / "groups.json").write_text(json.dumps(groups))
    files = {k: {"path": n, "sha256": sha256_file(directory / n)} for k, n in (("tokens", "tokens.npy"), ("offsets", "offsets.npy"), ("groups", "groups.json"))}
    atomic_write_json(directory / "manifest.json", {"format": FORMAT, "tokenizer_files": tokenizer_files, "files": files,
                                                     "documents": len(documents), "tokens": int(len(tokens))})
    return directory / "manifest.json"


class MixtureWindows:
    def __init__(self, sources: list[Source], length: int, *, tokenizer_files: dict[str, str], vocab_size: int, heldout_fraction: float = 0.1,
                 split_seed: int = 42):
        if length < 2 or not 0 < heldout_fraction < 1 or vocab_size < 1:
            raise ValueError("invalid document-window contract")
        if not sources:
            raise ValueError("empty corpus")
        self.length, self.parts, self.receipts = length, [], []
        weights = np.asarray([s.weight for s in sources], dtype=np.float64)
        self.weights = weights / weights.sum()
        for source in sources:
            path = Path(source.manifest).resolve(strict=True)
            manifest = json.loads(path.read_text())
            if manifest.get("format") != FORMAT:
                raise ValueError("unsupported corpus format; bare token files are not accepted")
            if manifest.get("tokenizer_files") != tokenizer_files:
                raise ValueError(f"tokenizer identity differs from the model's: {path}")
            assets = {}
            for key in ("tokens", "offsets", "groups"):
                record = manifest["files"][key]
                asset = (path.parent / record["path"]).resolve(strict=True)
                if not asset.is_relative_to(path.parent) or sha256_file(asset) != record["sha256"]:
                    raise ValueError(f"corpus asset escapes its source or its checksum differs: {key}")
                assets[key] = asset
            tokens = np.load(assets["tokens"], mmap_mode="r", allow_pickle=False)
            offsets = np.load(assets["offsets"], mmap_mode="r", allow_pickle=False)
            groups = json.loads(assets["groups"].read_text())
            integer = (np.dtype("int32"), np.dtype("int64"))
            if tokens.ndim != 1 or tokens.dtype not in integer or offsets.ndim != 1 or offsets.dtype not in integer:
                raise ValueError("tokens and offsets must be one-dimensional int32 / int64 arrays")
            if len(offsets) < 2 or offsets[0] != 0 or offsets[-1] != len(tokens) or np.any(np.diff(offsets) <= 0):
                raise ValueError("offsets must partition every token into non-empty documents")
            if not isinstance(groups, list) or len(groups) != len(offsets) - 1 or any(not isinstance(g, str) or not g for g in groups):
                raise ValueError("one non-empty stable group id is required per document")
            for start in range(0, len(tokens), 1 << 20):
                block = tokens[start:start + (1 << 20)]
                if block.min() < 0 or block.max() >= vocab_size:
                    raise ValueError("a corpus token id is outside the vocabulary")
            lengths = np.diff(offsets)
            picks = {False: [], True: []}
            for i, g in enumerate(groups):
                if lengths[i] >= length:
                    picks[heldout_group(g, split_seed, heldout_fraction)].append(i)
            if not picks[False] or not picks[True]:
                raise ValueError("each source needs eligible documents in both the train and the held-out set")
            self.parts.append((tokens, offsets, {k: np.asarray(v) for k, v in picks.items()}))
            self.receipts.append({"manifest": str(path), "sha256": sha256_file(path), "weight": source.weight, "train_documents": len(picks[False]),
                                  "heldout_documents": len(picks[True]), "short_documents": len(groups) - len(picks[False]) - len(picks[True])})

    def sample(self, rng: np.random.Generator, count: int, *, heldout: bool = False) -> torch.Tensor:
        if count < 1:
            raise ValueError("sample count must be positive")
        out = np.empty((count, self.length), dtype=np.int64)
        for row, s in enumerate(rng.choice(len(self.parts), size=count, p=self.weights)):
            tokens, offsets, picks = self.parts[s]
            doc = int(picks[heldout][int(rng.integers(len(picks[heldout])))])
            lo, hi = int(offsets[doc]), int(offsets[doc + 1])
            start = int(rng.integers(lo, hi - self.length + 1))
            out[row] = tokens[start:start + self.length]
        return torch.from_numpy(out)

    def rank_batch(self, seed: int, step: int, rank: int, per_rank: int, *, heldout: bool = False) -> torch.Tensor:
        """The windows of ``rank`` at ``step``: a function of (seed, step, rank) only, so a resumed run or the other arm of
        a comparison sees the same data without replaying a generator."""
        return self.sample(np.random.default_rng([seed, step, rank, int(heldout)]), per_rank, heldout=heldout)
