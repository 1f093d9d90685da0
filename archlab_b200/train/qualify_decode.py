"""Independent controls for fixed-cache decoding of a Limite model: is the cached arithmetic the model's arithmetic, and
do graph replay and cache migration reproduce the eager fixed-cache path EXACTLY?

Two different questions with two different standards.  (a) Cached decoding against the full forward: a tolerance,
because the reduction order differs.  (b) The ``GraphDecoder`` (captured on CUDA, eager elsewhere) and a migrated cache
against the eager fixed-cache implementation: bit equality of every logit and of every logical cache entry -- a
difference here is an indexing error, never "bf16 noise".

* ``cache_equal``: same geometry, same position, equal tensors layer by layer.
* ``select_rows(cache, rows, length)``: a new cache holding the chosen batch rows (requests that go on after others
  finished), ``cache_selection_equal`` checks it against the unmigrated tensors without using ``select_rows``' own
  indexing: per layer the visible window of every chosen row matches and nothing else is populated.
* ``fixed_cache_decode_controls``: prefill, then ``steps`` tokens (teacher-forced from ``ids`` or greedy) through all
  three paths; returns the worst deviations and raises on an exactness violation.
(Reference: src/archlab/qualification/limite_decode.py:15-170.)
"""
from __future__ import annotations

import torch

from ..models.limite import GraphDecoder, LimiteLM, StaticDecodeCache, decode_step, prefill


def cache_equal(a: StaticDecodeCache, b: StaticDecodeCache) -> bool:
    if a.sizes != b.sizes or a.capacity != b.capacity or not torch.equal(a.position, b.position):
        return False
    return all(x.shape == y.shape and x.dtype == y.dtype and torch.equal(x, y) for x, y in zip((*a.k, *a.v), (*b.k, *b.v)))


def select_rows(cache: StaticDecodeCache, rows: torch.Tensor) -> StaticDecodeCache:
    out = StaticDecodeCache(cache.c, len(rows), cache.capacity, cache.position.device, cache.k[0].dtype)
    for i in range(len(cache.k)):
        out.k[i].copy_(cache.k[i][rows])
        out.v[i].copy_(cache.v[i][rows])
    out.position.copy_(cache.position)
    return out


def cache_selection_equal(source: StaticDecodeCache, selected: StaticDecodeCache, rows: torch.Tensor) -> bool:
    """Checked slot by slot against the source: the slots a token at ``position`` can see must match the chosen source
    row, every other slot must be empty."""
    if source.sizes != selected.sizes or not torch.equal(source.position, selected.position):
        return False
    length = int(source.position)
    for layer, n in enumerate(source.sizes):
        visible = torch.zeros(n, dtype=torch.bool, device=source.position.device)
        visible[[p % n for p in range(max(0, length - n), length)]] = True
        for src, dst in ((source.k[layer], selected.k[layer]), (source.v[layer], selected.v[layer])):
            for out_row, src_row in enumerate(rows.tolist()):
                if not torch.equal(dst[out_row][visible], src[src_row][visible]):
                    return False
                if bool(dst[out_row][~visible].count_nonzero()) and not torch.equal(dst[out_row][~visible], src[src_row][~visible]):
                    return False
    return True


@torch.no_grad()
def fixed_cache_decode_controls(model: LimiteLM, ids: torch.Tensor, capacity: int, *, steps: int = 8, teacher_forcing: bool = True,
                                tolerance: float = 2e-3) -> dict:
    """``ids`` [B, T + steps] when teacher-forced (the first T tokens are the prompt), [B, T] when greedy."""
    if model.training:
        raise ValueError("decode qualification needs eval mode")
    B = ids.size(0)
    T = ids.size(1) - steps if teacher_forcing else ids.size(1)
    if T < 1 or T + steps > capacity:
        raise ValueError("prompt and steps must fit the cache capacity")
    logits, ks, vs = prefill(model, ids[:, :T])
    p = next(model.parameters())
    eager = StaticDecodeCache(model.config, B, capacity, p.device, p.dtype)
    eager.load_prefill(ks, vs)
    decoder = GraphDecoder(model, B, capacity)
    first = ids[:, T:T + 1] if teacher_forcing else logits.argmax(-1, keepdim=True)
    decoder.reset(ks, vs, first)
    history, token = ids[:, :T], first
    worst_full, exact = 0.0, True
    for step in range(steps):
        history = torch.cat((history, token), 1)
        a = decode_step(model, eager, token)
        b = decoder(token).clone()
        full = model(history)[:, -1].float()
        worst_full = max(worst_full, float((a - full).abs().max()))
        exact = exact and torch.equal(a, b) and cache_equal(eager, decoder.cache)
        token = ids[:, T + step + 1:T + step + 2] if teacher_forcing and step + 1 < steps else a.argmax(-1, keepdim=True)
    if not exact:
        raise AssertionError("the decoder diverged from the eager fixed-cache path: an indexing or capture error")
    if worst_full > tolerance:
        raise AssertionError(f"cached decoding deviates from the full forward by {worst_full:.3e} (tolerance {tolerance:.1e})")
    rows = torch.arange(B - 1, -1, -1, device=p.device)          # a full permutation: same kernel shapes, every row moves
    moved = select_rows(eager, rows)
    if not cache_selection_equal(eager, moved, rows):
        raise AssertionError("cache migration changed a visible entry")
    follow = decode_step(model, moved, token[rows])
    reference = decode_step(model, eager, token)[rows]
    if not torch.equal(follow, reference):
        raise AssertionError("decoding after cache migration differs from the unmigrated rows")
    return {"steps": steps, "batch": B, "prompt_tokens": T, "max_abs_error_vs_full_forward": worst_full, "decoder_bitwise_equal": True,
            "migration_bitwise_equal": True, "captured": decoder.graph is not None}
