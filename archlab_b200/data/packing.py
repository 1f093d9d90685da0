"""BOS-aligned best-fit packing (src/archlab/speedrun/dataloader.py:154-276).

Every row holds ``T + 1`` tokens and starts with BOS.  For each row: repeatedly take, from a buffer
of tokenised documents, the LARGEST document that still fits; when none fits, crop the SHORTEST
buffered document to fill the row exactly.  100 % utilisation (no padding).  The packer is a pure
function of the document stream, so a resumed run replays to its exact ``batch_index``; in
"replicated global batch" mode every rank rebuilds the canonical one-rank stream and slices it,
padding with ``-1`` targets when the world size does not divide the batch
(src/archlab/speedrun/dataloader.py:286-359).
"""
from __future__ import annotations

from collections.abc import Iterable, Iterator

import torch


class BestFitPacker:
    def __init__(self, documents: Iterable[list[int]], batch_size: int, seq_len: int, *, buffer_size: int = 1000,
                 bos_token: int | None = None):
        """``documents`` yields token lists; when ``bos_token`` is given it is prepended to each."""
        self.docs: Iterator[list[int]] = iter(documents)
        self.B, self.T = batch_size, seq_len
        self.buffer_size = buffer_size
        self.bos = bos_token
        self.buffer: list[list[int]] = []
        self.batch_index = 0

    def _refill(self) -> None:
        while len(self.buffer) < self.buffer_size:
            doc = next(self.docs)
            if self.bos is not None:
                doc = [self.bos, *doc]
            if doc:
                self.buffer.append(doc)

    def _row(self) -> list[int]:
        cap = self.T + 1
        row: list[int] = []
        while len(row) < cap:
            self._refill()
            remaining = cap - len(row)
            best, best_len = -1, 0
            for i, d in enumerate(self.buffer):
                if best_len < len(d) <= remaining:
                    best, best_len = i, len(d)
            if best >= 0:
                row.extend(self.buffer.pop(best))
            else:
                shortest = min(range(len(self.buffer)), key=lambda i: len(self.buffer[i]))
                row.extend(self.buffer.pop(shortest)[:remaining])
        return row

    def next_batch(self) -> tuple[torch.Tensor, torch.Tensor, dict]:
        rows = torch.tensor([self._row() for _ in range(self.B)], dtype=torch.long)
        state = {"batch_index": self.batch_index}
        self.batch_index += 1
        return rows[:, :-1].contiguous(), rows[:, 1:].contiguous(), state

    def __iter__(self):
        return self

    def __next__(self):
        return self.next_batch()

    def seek(self, batch_index: int) -> None:
        """Deterministic replay to an exact batch cursor (rebuilds the buffered best-fit state)."""
        while self.batch_index < batch_index:
            self.next_batch()


def replicated_global_batch(packer: BestFitPacker, rank: int, world_size: int):
    """Slice the canonical one-rank stream: rank r takes rows ``r::world``-contiguous blocks; rows
    added to make the batch divisible carry ``-1`` targets so they contribute no loss."""
    x, y, state = packer.next_batch()
    B = x.size(0)
    per = -(-B // world_size)
    pad = per * world_size - B
    if pad:
        x = torch.cat([x, x[:pad]], dim=0)
        y = torch.cat([y, torch.full_like(y[:pad], -1)], dim=0)
    return x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per], state


def balanced_slice(global_batch: int, rank: int, world_size: int) -> tuple[int, int, int]:
    """``(start, active, local_size)`` of one rank's share of an exact global batch.  Every rank gets the same static
    shape ``ceil(global / world)``; when the world does not divide the batch the first ``global % world`` ranks hold one
    more ACTIVE row than the rest and the others carry one ignored row, so no rank idles on several padded rows while
    another is full (192 sequences on 15 ranks: twelve ranks with 13 active rows, three with 12, all of shape 13).
    Active rows stay contiguous in the canonical one-rank stream (src/archlab/speedrun/dataloader.py:286-306)."""
    if global_batch <= 0:
        raise ValueError("global_batch must be positive")
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must lie inside a positive world size")
    base, extra = divmod(global_batch, world_size)
    return rank * base + min(rank, extra), base + (rank < extra), base + (extra > 0)


def balanced_global_batch(packer: BestFitPacker, rank: int, world_size: int):
    """Like ``replicated_global_batch`` with the balanced split: ignored rows repeat the rank's first row with ``-1``
    targets, so shapes are static and the loss sees exactly the global batch."""
    x, y, state = packer.next_batch()
    start, active, local = balanced_slice(x.size(0), rank, world_size)
    xs, ys = x[start:start + active], y[start:start + active]
    if active < local:
        xs = torch.cat([xs, xs[:local - active]], dim=0)
        ys = torch.cat([ys, torch.full_like(ys[:local - active], -1)], dim=0)
    return xs, ys, {**state, "active_rows": active}


def tokenizing_loader(data_dir, tokenizer, batch_size: int, seq_len: int, *, split: str = "train", rank: int = 0, world: int = 1,
                      buffer_size: int = 1000, resume_state: dict | None = None, bos_token: int | None = None):
    """Parquet shards -> tokenizer -> best-fit packer, yielding ``(inputs, targets, state)``.

    ``state`` = ``{"batch_index", "shard", "row_group", "epoch"}``: the batch cursor plus the position of the document
    stream when the batch was cut (for logs and sanity checks).  Resuming is EXACT: the packer's buffer contents are a
    function of the whole document stream, so ``resume_state`` replays the stream to ``batch_index`` (tokenising again,
    discarding batches) instead of guessing the buffer from a file cursor; the first batch after a resume is the batch
    that was in flight when the state was saved (src/archlab/speedrun/dataloader.py:154-276)."""
    from .parquet_shards import document_batches

    cursor = {"shard": 0, "row_group": 0, "epoch": 1}
    if bos_token is None:
        bos_token = getattr(tokenizer, "special", {}).get("<|bos|>") if hasattr(tokenizer, "special") else None

    def documents():
        for texts, (shard, group, epoch) in document_batches(data_dir, split, rank=rank, world=world):
            cursor.update(shard=shard, row_group=group, epoch=epoch)
            for text in texts:
                yield tokenizer.encode(text)

    packer = BestFitPacker(documents(), batch_size, seq_len, buffer_size=buffer_size, bos_token=bos_token)
    if resume_state is not None:
        packer.seek(int(resume_state["batch_index"]))
    while True:
        x, y, state = packer.next_batch()
        yield x, y, {**state, **cursor}
