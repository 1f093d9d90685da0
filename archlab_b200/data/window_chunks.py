"""Pre-training chunks in which every target token is predicted exactly once.

A document ``[BOS, t1 .. tn, EOD]`` is cut into windows of at most ``sequence`` TARGETS: window k takes inputs
``tokens[s : s + c]`` and targets ``tokens[s + 1 : s + c + 1]`` with ``s = k * sequence``, so consecutive windows overlap
by one input token and no target is seen twice or skipped; windows never cross a document boundary (the short last
window of a document is padded with ignored targets when batched).  Per chunk of source rows the job writes

    tokens.u32     all documents back to back (little-endian uint32)
    windows.npy    [n, 3] uint64 rows: token offset of the window's first input, target count, running target index
    COMPLETE.json  counts, the SHA-256 of both files and of every document used, written last

Documents whose text hash is in ``exclude`` (a held-out or benchmark set) or that are empty are skipped; whole documents
are shuffled inside the chunk with a seed derived from the chunk index, so the order does not depend on which worker
ran the chunk.  A chunk whose ``COMPLETE.json`` exists is not redone.  ``ChunkReader`` verifies the receipt and serves
batches.  (Reference: src/archlab/preprocessing/v41_scratch.py:32-131.)
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Callable, Iterator

import numpy as np
import torch

from ..contracts.substrate import atomic_write_json, sha256_file

FORMAT = "archlab-document-chunk-v1"


def document_windows(length: int, sequence: int) -> Iterator[tuple[int, int]]:
    """(start, target count) of every window of a document of ``length`` tokens."""
    for start in range(0, length - 1, sequence):
        yield start, min(sequence, length - 1 - start)


def prepare_chunk(out_dir, split: str, index: int, texts: list[str], encode_batch: Callable[[list[str]], list[list[int]]], *, sequence: int,
                  bos: int = 0, eod: int = 1, exclude: frozenset[str] = frozenset(), base_seed: int = 2234, source: str = "") -> dict:
    out = Path(out_dir) / "chunks" / f"{split}-{index:06d}"
    out.mkdir(parents=True, exist_ok=True)
    if (out / "COMPLETE.json").exists():
        return json.loads((out / "COMPLETE.json").read_text())
    hashes = [hashlib.sha256(t.encode()).hexdigest() for t in texts]
    keep = [i for i, h in enumerate(hashes) if texts[i] and h not in exclude]
    order = np.random.default_rng(base_seed + index).permutation(keep).tolist()
    windows, used, offset, targets = [], [], 0, 0
    with (out / "tokens.u32.tmp").open("wb") as stream:
        for first in range(0, len(order), 128):
            batch = order[first:first + 128]
            for doc, ids in zip(batch, encode_batch([texts[i] for i in batch])):
                tokens = [bos, *ids, eod]
                stream.write(np.asarray(tokens, dtype="<u4").tobytes())
                used.append(hashes[doc])
                for start, count in document_windows(len(tokens), sequence):
                    windows.append((offset + start, count, targets))
                    targets += count
                offset += len(tokens)
    (out / "tokens.u32.tmp").replace(out / "tokens.u32")
    with (out / "windows.npy.tmp").open("wb") as stream:
        np.save(stream, np.asarray(windows, dtype="<u8").reshape(-1, 3), allow_pickle=False)
    (out / "windows.npy.tmp").replace(out / "windows.npy")
    receipt = {"format": FORMAT, "split": split, "index": index, "source": source, "documents": len(used), "document_sha256": used,
               "excluded_or_empty": len(texts) - len(used), "windows": len(windows), "targets": targets, "stored_tokens": offset, "sequence": sequence,
               "tokens_sha256": sha256_file(out / "tokens.u32"), "windows_sha256": sha256_file(out / "windows.npy")}
    atomic_write_json(out / "COMPLETE.json", receipt)
    return receipt


class ChunkReader:
    def __init__(self, chunk_dir, *, verify: bool = True):
        self.dir = Path(chunk_dir)
        self.receipt = json.loads((self.dir / "COMPLETE.json").read_text())
        if self.receipt.get("format") != FORMAT:
            raise ValueError("not a document chunk of this framework")
        if verify and (sha256_file(self.dir / "tokens.u32") != self.receipt["tokens_sha256"] or sha256_file(self.dir / "windows.npy") != self.receipt["windows_sha256"]):
            raise ValueError(f"chunk payload changed: {self.dir}")
        self.tokens = np.memmap(self.dir / "tokens.u32", dtype="<u4", mode="r")
        self.windows = np.load(self.dir / "windows.npy", allow_pickle=False)
        self.sequence = self.receipt["sequence"]
        if len(self.tokens) != self.receipt["stored_tokens"] or len(self.windows) != self.receipt["windows"]:
            raise ValueError("chunk counts differ from the receipt")

    def __len__(self) -> int:
        return len(self.windows)

    def batch(self, rows) -> tuple[torch.Tensor, torch.Tensor]:
        """(inputs, labels) [len(rows), sequence]; short windows are padded with input 0 and label -1."""
        x = np.zeros((len(rows), self.sequence), dtype=np.int64)
        y = np.full((len(rows), self.sequence), -1, dtype=np.int64)
        for r, w in enumerate(rows):
            start, count, _ = (int(v) for v in self.windows[w])
            x[r, :count] = self.tokens[start:start + count]
            y[r, :count] = self.tokens[start + 1:start + count + 1]
        return torch.from_numpy(x), torch.from_numpy(y)
