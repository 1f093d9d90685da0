"""Engram geometry under width scaling: channels and hash-bucket counts move with the model width, and every hash
head keeps its own prime bucket count.

Rule (src/archlab/architectures/engram_scaling.py:7-39; vectors in the reference's
tests/test_v41_performance_contract.py:7-20,95-103): with ratio = width / original hidden size (or the declared
``anchor_width`` / hidden size when a fixed lookup budget is wanted),

* channels per head = ceil(head_dim x ratio / 8) x 8, at least 8 (a kernel-aligned count instead of padded tensors);
* buckets = round(vocab x ratio), at least 2;
* every (layer, n-gram order, head) takes the next unused prime >= the previous head's prime + 1, starting again from
  ``buckets`` for every (layer, order); a layer's table holds the sum of its primes.
"""
from __future__ import annotations

from fractions import Fraction
from math import isqrt
from typing import Iterator, Mapping


def _is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n < 4:
        return True
    if n % 2 == 0:
        return False
    return all(n % d for d in range(3, isqrt(n) + 1, 2))


def _fresh_primes(start: int, taken: set[int]) -> Iterator[int]:
    """Primes >= start that nobody took yet, ascending; each one yielded is marked as taken."""
    n = start
    while True:
        if n not in taken and _is_prime(n):
            taken.add(n)
            yield n
        n += 1


def scaled_engram_geometry(original: Mapping, width: int, *, anchor_width: int | None = None) -> dict:
    if anchor_width is not None and (type(anchor_width) is not int or anchor_width <= 0):
        raise ValueError("Engram anchor width must be a positive integer")
    ratio = Fraction(anchor_width if anchor_width is not None else width, original["hidden_size"])
    exact_channels = original["engram_head_dim"] * ratio
    channels = max(8, 8 * -(-exact_channels.numerator // (8 * exact_channels.denominator)))
    buckets = max(2, round(original["engram_vocab_size"] * ratio))
    taken: set[int] = set()
    orders, heads = original["engram_max_ngram_size"] - 1, original["engram_n_heads"]
    tables = []
    for _layer in original["engram_layer_ids"]:
        rows = 0
        for _order in range(orders):
            source, last = None, buckets - 1
            for _head in range(heads):
                source = _fresh_primes(last + 1, taken)
                last = next(source)
                rows += last
        tables.append(rows)
    return {"engram_head_dim": int(channels), "engram_vocab_size": int(buckets), "engram_num_embeddings": tables}
