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
