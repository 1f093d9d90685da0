"""FineWeb ``.bin`` token shards (llm.c / modded-nanogpt format) with deterministic rank slicing.

File format (fixed by the published shards): 256 int32 header words (magic 20240520, version 1, token count),
then uint16 tokens.  Batch geometry (fixed by the reference's loader, src/archlab/fineweb.py:96-246, because a
resumed run must land on the same tokens): one distributed batch is one contiguous range of
``world x local_batch x T`` tokens inside a shard, cut into equal rank-local ranges, each read with one extra
trailing token so that labels are the inputs shifted by one; a shard is left as soon as it cannot supply a
whole distributed batch plus that one token, and the shard list wraps around.

Structure here: a ``ShardTable`` is built once from the headers (token count and number of whole batches per
shard, prefix sums over an epoch).  A batch index maps to (shard, offset) in closed form, so ``seek_batch`` touches
no payload and no shard in between, and the loader itself is a cursor over that table holding one memory map.
"""
from __future__ import annotations

import bisect
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

HEADER_INTS = 256
HEADER_BYTES = HEADER_INTS * 4
MAGIC = 20_240_520
VERSION = 1
TRAIN_SHARDS = 103                       # the complete published inventory: fineweb_train_000001 .. 000103


def write_fineweb_shard(path: str | Path, tokens) -> None:
    """Writer for tests and synthetic corpora."""
    payload = np.ascontiguousarray(tokens, dtype=np.uint16)
    head = struct.pack("<3i", MAGIC, VERSION, payload.size) + bytes(HEADER_BYTES - 12)
    Path(path).write_bytes(head + payload.tobytes())


def inspect_fineweb_shard(path) -> int:
    """Token count of a shard after checking header and file length."""
    path = Path(path)
    with path.open("rb") as f:
        head = f.read(HEADER_BYTES)
    if len(head) < HEADER_BYTES:
        raise ValueError(f"{path}: header is shorter than {HEADER_BYTES} bytes")
    magic, version, count = struct.unpack_from("<3i", head)
    problems = []
    if magic != MAGIC:
        problems.append(f"magic {magic} != {MAGIC}")
    elif version != VERSION:
        problems.append(f"version {version} is not supported")
    elif path.stat().st_size != HEADER_BYTES + 2 * count:
        problems.append(f"length {path.stat().st_size} does not match {count} tokens")
    if problems:
        raise ValueError(f"{path}: {problems[0]}")
    return count


def _shard_number(path: Path) -> int:
    return int(path.stem.rsplit("_", 1)[1])


def inspect_fineweb_dataset(root, *, expected_train_shards: int = TRAIN_SHARDS, required_train_tokens: int | None = None) -> dict:
    """Inventory check before a run.  Without ``required_train_tokens`` the complete numbered inventory must be
    present; with it, the numbered prefix 1, 2, ... is validated until it holds that many tokens."""
    root = Path(root)
    train = {_shard_number(p): p for p in root.glob("fineweb_train_*.bin")}
    val = sorted(p.name for p in root.glob("fineweb_val_*.bin"))
    if not train:
        raise ValueError(f"{root}: no train shards")
    if val != ["fineweb_val_000000.bin"]:
        raise ValueError(f"{root}: the validation split must be exactly fineweb_val_000000.bin, found {val}")
    if required_train_tokens is None and len(train) != expected_train_shards:
        raise ValueError(f"{root}: {len(train)} train shards visible, the complete inventory has {expected_train_shards}")
    wanted = required_train_tokens or 0
    last = expected_train_shards if not wanted else max(train)
    counted = tokens = 0
    for number in range(1, last + 1):
        if number not in train:
            raise ValueError(f"{root}: train shard {number:06d} is missing")
        tokens += inspect_fineweb_shard(train[number])
        counted += 1
        if wanted and tokens >= wanted:
            break
    if tokens < wanted:
        raise ValueError(f"{root}: the shard prefix holds {tokens} tokens, {wanted} are required")
    return {"visible_train_shards": len(train), "validated_train_shards": counted, "validation_shards": len(val),
            "validated_train_tokens": tokens, "validation_tokens": inspect_fineweb_shard(root / val[0]),
            "complete_inventory": len(train) == expected_train_shards}


@dataclass(frozen=True)
class ShardTable:
    """Headers of a split and the batch arithmetic over them."""
    paths: tuple[Path, ...]
    tokens: tuple[int, ...]
    batch_tokens: int                     # tokens of one distributed batch
    batches: tuple[int, ...]              # whole batches each shard supplies (one spare token for the labels)
    first_batch: tuple[int, ...]          # epoch-relative index of each shard's first batch

    @classmethod
    def scan(cls, root, split: str, batch_tokens: int) -> "ShardTable":
        paths = tuple(sorted(Path(root).glob(f"fineweb_{split}_*.bin")))
        if not paths:
            raise FileNotFoundError(f"no FineWeb {split} shards under {Path(root)}")
        tokens = tuple(inspect_fineweb_shard(p) for p in paths)
        batches = tuple(max(0, (n - 1) // batch_tokens) for n in tokens)
        if not any(batches):
            raise ValueError("no shard is large enough for one distributed batch")
        starts, run = [], 0
        for b in batches:
            starts.append(run)
            run += b
        return cls(paths, tokens, batch_tokens, batches, tuple(starts))

    @property
    def epoch_batches(self) -> int:
        return self.first_batch[-1] + self.batches[-1]

    def locate(self, batch_index: int) -> tuple[int, int]:
        """(shard, token offset of the batch inside it) of the ``batch_index``-th batch from the start."""
        within = batch_index % self.epoch_batches
        shard = bisect.bisect_right(self.first_batch, within) - 1
        while self.batches[shard] == 0:                 # shards too small for a batch sort equal to their successor
            shard -= 1
        return shard, (within - self.first_batch[shard]) * self.batch_tokens


class FineWebBinaryLoader:
    """Iterator over this rank's ``(inputs, labels)`` of successive distributed batches."""

    def __init__(self, root, split: str, local_batch_size: int, sequence_length: int, *, rank: int, world_size: int,
                 device="cuda", start_batch_index: int = 0):
        if split not in ("train", "val"):
            raise ValueError("split must be 'train' or 'val'")
        for name, value in (("local_batch_size", local_batch_size), ("sequence_length", sequence_length), ("world_size", world_size)):
            if value <= 0:
                raise ValueError(f"{name} must be positive")
        if not 0 <= rank < world_size:
            raise ValueError("rank must lie inside the world size")
        self.local_batch_size, self.sequence_length = local_batch_size, sequence_length
        self.rank, self.world_size = rank, world_size
        self.local_tokens = local_batch_size * sequence_length
        self.global_tokens = self.local_tokens * world_size
        self.table = ShardTable.scan(root, split, self.global_tokens)
        self.files = list(self.table.paths)
        self.device = torch.device(device)
        self._mapped = (-1, None)
        self.seek_batch(start_batch_index)

    # -- cursor --------------------------------------------------------------------------------------
    def seek_batch(self, batch_index: int) -> None:
        if batch_index < 0:
            raise ValueError("batch index must be non-negative")
        self.batch_index = batch_index
        self.shard_index, self.global_position = self.table.locate(batch_index)

    def state_dict(self) -> dict[str, int]:
        return {"shard_index": self.shard_index, "global_position": self.global_position, "batch_index": self.batch_index}

    def _payload(self, shard: int) -> np.memmap:
        if self._mapped[0] != shard:
            self._mapped = (shard, np.memmap(self.table.paths[shard], dtype=np.uint16, mode="r", offset=HEADER_BYTES,
                                             shape=(self.table.tokens[shard],)))
        return self._mapped[1]

    # -- reading -------------------------------------------------------------------------------------
    def next_block(self) -> torch.Tensor:
        """This rank's ``local_tokens + 1`` int64 ids of the current batch; advances the cursor."""
        lo = self.global_position + self.rank * self.local_tokens
        ids = self._payload(self.shard_index)[lo:lo + self.local_tokens + 1].astype(np.int64)
        self.seek_batch(self.batch_index + 1)
        return torch.from_numpy(ids)

    def __iter__(self):
        return self

    def __next__(self):
        block = self.next_block()
        shape = (self.local_batch_size, self.sequence_length)
        x, y = block[:-1].view(shape), block[1:].view(shape)
        if self.device.type == "cuda":
            return x.pin_memory().to(self.device, non_blocking=True), y.pin_memory().to(self.device, non_blocking=True)
        return x.to(self.device), y.to(self.device)


def fixed_fineweb_validation_loader(root, local_batch_size: int, sequence_length: int, *, window_batches: int,
                                    rank: int = 0, world_size: int = 1, device="cuda"):
    """Endless generator that replays the same first ``window_batches`` validation batches at every evaluation."""
    if window_batches < 1:
        raise ValueError("window_batches must be positive")
    loader = FineWebBinaryLoader(root, "val", local_batch_size, sequence_length, rank=rank, world_size=world_size, device=device)
    while True:
        loader.seek_batch(0)
        for _ in range(window_batches):
            yield next(loader)
