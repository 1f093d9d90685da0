"""FineWeb ``.bin`` token shards (llm.c / modded-nanogpt format) with deterministic rank slicing.

File format: 256 int32 header words (magic 20240520, version 1, token count), then uint16 tokens.
One global batch is one contiguous token range split into equal rank-local ranges; each range
carries one extra trailing token so labels are the inputs shifted by one.  ``seek_batch(i)``
reaches an exact distributed-batch cursor without reading payloads, which is how a resumed run
derives its data position from the restored iteration.  Behaviour follows
src/archlab/fineweb.py:16-246.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

HEADER_INTS = 256
HEADER_BYTES = HEADER_INTS * 4
MAGIC = 20_240_520
VERSION = 1


def write_fineweb_shard(path: str | Path, tokens: np.ndarray) -> None:
    """Writer for tests and synthetic corpora."""
    tokens = np.asarray(tokens, dtype=np.uint16)
    header = np.zeros(HEADER_INTS, dtype=np.int32)
    header[0], header[1], header[2] = MAGIC, VERSION, tokens.size
    with Path(path).open("wb") as f:
        f.write(header.tobytes())
        f.write(tokens.tobytes())


def inspect_fineweb_shard(path: Path) -> int:
    with Path(path).open("rb") as f:
        raw = f.read(HEADER_BYTES)
    if len(raw) != HEADER_BYTES:
        raise ValueError(f"truncated FineWeb header: {path}")
    header = np.frombuffer(raw, dtype=np.int32)
    if int(header[0]) != MAGIC:
        raise ValueError(f"FineWeb magic mismatch in {path}")
    if int(header[1]) != VERSION:
        raise ValueError(f"unsupported FineWeb shard version in {path}: {int(header[1])}")
    n = int(header[2])
    if Path(path).stat().st_size != HEADER_BYTES + 2 * n:
        raise ValueError(f"FineWeb shard length mismatch in {path}: {Path(path).stat().st_size} != {HEADER_BYTES + 2 * n}")
    return n


def inspect_fineweb_dataset(root, *, expected_train_shards: int = 103, required_train_tokens: int | None = None) -> dict:
    root = Path(root)
    train = sorted(root.glob("fineweb_train_*.bin"))
    val = sorted(root.glob("fineweb_val_*.bin"))
    if not train:
        raise ValueError("FineWeb has no visible train shards")
    if val != [root / "fineweb_val_000000.bin"]:
        raise ValueError("FineWeb requires exactly fineweb_val_000000.bin")
    if required_train_tokens is None and len(train) != expected_train_shards:
        raise ValueError(f"complete FineWeb inventory requires {expected_train_shards} train shards; found {len(train)}")
    need = required_train_tokens or 0
    paths = ([root / f"fineweb_train_{i:06d}.bin" for i in range(1, expected_train_shards + 1)] if need == 0 else train)
    tokens = validated = 0
    for idx, p in enumerate(paths, start=1):
        if p.name != f"fineweb_train_{idx:06d}.bin" or not p.is_file():
            raise ValueError(f"FineWeb is missing required train shard {idx:06d}")
        tokens += inspect_fineweb_shard(p)
        validated += 1
        if need and tokens >= need:
            break
    if tokens < need:
        raise ValueError(f"FineWeb prefix has {tokens} validated tokens, fewer than the required {need}")
    return {"visible_train_shards": len(train), "validated_train_shards": validated, "validation_shards": len(val),
            "validated_train_tokens": tokens, "validation_tokens": sum(inspect_fineweb_shard(p) for p in val),
            "complete_inventory": len(train) == expected_train_shards}


class FineWebBinaryLoader:
    def __init__(self, root, split: str, local_batch_size: int, sequence_length: int, *, rank: int, world_size: int,
                 device="cuda", start_batch_index: int = 0):
        if split not in {"train", "val"}:
            raise ValueError("split must be 'train' or 'val'")
        if local_batch_size <= 0 or sequence_length <= 0:
            raise ValueError("batch size and sequence length must be positive")
        if world_size <= 0 or not 0 <= rank < world_size:
            raise ValueError("rank must be inside a positive world size")
        if start_batch_index < 0:
            raise ValueError("start batch index must be non-negative")
        self.files = sorted(Path(root).glob(f"fineweb_{split}_*.bin"))
        if not self.files:
            raise FileNotFoundError(f"no FineWeb {split} shards under {Path(root)}")
        self.local_batch_size, self.sequence_length = local_batch_size, sequence_length
        self.local_tokens = local_batch_size * sequence_length
        self.global_tokens = self.local_tokens * world_size
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device)
        self.shard_index = self.global_position = self.batch_index = 0
        self.tokens = None
        self.token_count = 0
        self._open()
        if not any(inspect_fineweb_shard(p) > self.global_tokens for p in self.files):
            raise ValueError("no FineWeb shard is large enough for one distributed batch")
        self.seek_batch(start_batch_index)

    def _open(self) -> None:
        p = self.files[self.shard_index]
        self.token_count = inspect_fineweb_shard(p)
        self.tokens = np.memmap(p, dtype=np.uint16, mode="r", offset=HEADER_BYTES, shape=(self.token_count,))
        self.global_position = 0

    def _advance(self) -> None:
        self.shard_index = (self.shard_index + 1) % len(self.files)
        self._open()

    def seek_batch(self, batch_index: int) -> None:
        if batch_index < 0:
            raise ValueError("batch index must be non-negative")
        self.shard_index = 0
        self._open()
        self.batch_index = 0
        remaining = batch_index
        while remaining:
            available = max(0, (self.token_count - self.global_position - 1) // self.global_tokens)
            if remaining < available:
                self.global_position += remaining * self.global_tokens
                self.batch_index += remaining
                return
            remaining -= available
            self.batch_index += available
            self._advance()

    def state_dict(self) -> dict[str, int]:
        return {"shard_index": self.shard_index, "global_position": self.global_position,
                "batch_index": self.batch_index}

    def __iter__(self):
        return self

    def next_block(self) -> torch.Tensor:
        """This rank's ``[local_batch, T + 1]``-equivalent flat block (local_tokens + 1 int64 ids)."""
        while self.global_position + self.global_tokens + 1 > self.token_count:
            self._advance()
        start = self.global_position + self.rank * self.local_tokens
        buf = torch.from_numpy(np.array(self.tokens[start:start + self.local_tokens + 1], dtype=np.int64, copy=True))
        self.global_position += self.global_tokens
        self.batch_index += 1
        return buf

    def __next__(self):
        buf = self.next_block()
        x = buf[:-1].view(self.local_batch_size, self.sequence_length)
        y = buf[1:].view(self.local_batch_size, self.sequence_length)
        if self.device.type == "cuda":
            return x.pin_memory().to(self.device, non_blocking=True), y.pin_memory().to(self.device, non_blocking=True)
        return x.to(self.device), y.to(self.device)


def fixed_fineweb_validation_loader(root, local_batch_size: int, sequence_length: int, *, window_batches: int,
                                    rank: int = 0, world_size: int = 1, device="cuda"):
    """Replays the identical first ``window_batches`` validation batches at every evaluation."""
    if window_batches < 1:
        raise ValueError("window_batches must be positive")
    while True:
        loader = FineWebBinaryLoader(root, "val", local_batch_size, sequence_length, rank=rank,
                                     world_size=world_size, device=device)
        for _ in range(window_batches):
            yield next(loader)
