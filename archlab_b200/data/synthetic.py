"""Synthetic token streams for benchmarks and tests (the reference ships none; its loaders read
FineWeb shards).  Zipf(s) ids over the vocabulary from a fixed seed, or uniform ids; labels are the
inputs shifted by one, so a block is ``[batch, T + 1]``.
"""
from __future__ import annotations

import numpy as np
import torch


def zipf_probabilities(vocab_size: int, s: float = 1.1) -> np.ndarray:
    ranks = np.arange(1, vocab_size + 1, dtype=np.float64)
    p = ranks ** (-s)
    return p / p.sum()


class ZipfTokens:
    """Deterministic Zipf(s) token blocks: block ``i`` of rank ``r`` depends only on (seed, r, i)."""

    def __init__(self, vocab_size: int, seq_len: int, batch: int, *, s: float = 1.1, seed: int = 0,
                 rank: int = 0, pin: bool = False):
        self.vocab_size, self.seq_len, self.batch = vocab_size, seq_len, batch
        self.seed, self.rank, self.pin = seed, rank, pin
        self.cdf = np.cumsum(zipf_probabilities(vocab_size, s))
        self.cdf[-1] = 1.0

    def block(self, index: int) -> torch.Tensor:
        rng = np.random.default_rng([self.seed, self.rank, index])
        u = rng.random((self.batch, self.seq_len + 1))
        ids = np.searchsorted(self.cdf, u, side="right").astype(np.int64)
        np.minimum(ids, self.vocab_size - 1, out=ids)
        t = torch.from_numpy(ids)
        if self.pin and torch.cuda.is_available():
            t = t.pin_memory()
        return t


def uniform_tokens(vocab_size: int, seq_len: int, batch: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab_size, (batch, seq_len + 1), generator=g, dtype=torch.int64)
