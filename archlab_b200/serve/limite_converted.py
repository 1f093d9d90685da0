"""Serving a converted Limite model (2-simplicial attention in every layer) from paged caches.

Every layer owns one ``PagedSimplicialCache``: short keys / values (k1 = 1 + dK(h), v1 = 1 + dV(h)) and long keys /
values (the native k, v) of all live requests in 128-position pages.  The server admits exactly two kinds of work, and
keeps no request state outside the caches and the page tables:

* ``prefill(request, ids)``: one COMPLETE new prompt.  The model's training-form forward runs once (the tcgen05
  simplicial kernel on bf16 CUDA), and the per-layer operands are written to the request's pages.
* ``decode(requests, tokens)``: one new token for each of a batch of live requests.  Projections use every request's own
  position; the reduction is the paged decode kernel (``ops.simplicial_decode``) over the request's page list.

``validate_serving`` refuses settings whose paging or execution semantics this path does not implement (chunked prefill,
prefix sharing, quantised caches, speculative decoding, tensor / pipeline splits, an unconverted or adapter-carrying
model).  (Reference: the cache bridge into an external engine, src/archlab/training/serving_conversion.py:19-46,
135-240.)
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..models.blocks import rope_tables
from ..models.limite import LimiteLM, LimiteSimplicialAttention
from ..ops import block_ops
from ..ops.simplicial_decode import PAGE, PagedSimplicialCache, simplicial_decode


@dataclass(frozen=True)
class ServingSettings:
    tensor_parallel: int = 1
    pipeline_parallel: int = 1
    chunked_prefill: bool = False
    prefix_caching: bool = False
    cache_dtype: str = "auto"
    speculative: bool = False
    quantization: str | None = None


def validate_serving(model: LimiteLM, settings: ServingSettings, *, short_window: int | None = None) -> None:
    if settings.tensor_parallel != 1 or settings.pipeline_parallel != 1:
        raise ValueError("converted serving runs on one GPU per replica (TP = PP = 1)")
    if settings.chunked_prefill:
        raise ValueError("converted serving admits one complete prompt at a time (no chunked prefill)")
    if settings.prefix_caching or settings.cache_dtype not in ("auto", "bfloat16", "float16", "float32"):
        raise ValueError("converted serving needs private, unquantised K/V pages")
    if settings.quantization is not None or settings.speculative:
        raise ValueError("converted serving does not admit quantisation or speculative decoding")
    layers = [b.attn for b in model.layers]
    if not all(isinstance(a, LimiteSimplicialAttention) for a in layers) or any(b.prelude is not None for b in model.layers):
        raise ValueError("converted serving needs the attention replacement in every layer and no adapters")
    if short_window is not None and any(a.conversion.short_window != short_window for a in layers):
        raise ValueError(f"converted serving was qualified for short window {short_window}")


@dataclass
class _Request:
    length: int
    pages: list[int] = field(default_factory=list)


class ConvertedLimiteServer:
    def __init__(self, model: LimiteLM, *, num_pages: int, max_context: int, settings: ServingSettings = ServingSettings(), dtype=None):
        validate_serving(model, settings)
        if model.training:
            raise ValueError("serving needs eval mode")
        self.model, self.c, self.max_context = model, model.config, max_context
        dev = model.embed.weight.device
        dtype = dtype or model.embed.weight.dtype
        self.caches = [PagedSimplicialCache(num_pages, self.c.num_key_value_heads, self.c.head_dim, dev, dtype) for _ in model.layers]
        self.max_pages = -(-max_context // PAGE)
        self.requests: dict[str, _Request] = {}

    # every layer's cache hands out the same page numbers in the same order, so one page list serves all layers
    def _allocate(self, positions: int) -> list[int]:
        lists = [cache.allocate(positions) for cache in self.caches]
        if any(l != lists[0] for l in lists):
            raise RuntimeError("per-layer page tables diverged")
        return lists[0]

    def release(self, request: str) -> None:
        r = self.requests.pop(request)
        for cache in self.caches:
            cache.release(list(r.pages))

    def _windows(self, attn) -> tuple[int, int]:
        w2 = self.max_pages * PAGE if attn.native.is_global else self.c.window_span
        return min(attn.conversion.short_window, w2), w2

    @torch.inference_mode()
    def prefill(self, request: str, ids: torch.Tensor) -> torch.Tensor:
        """ids [T] -> logits of the last position [vocab] (fp32)."""
        if request in self.requests:
            raise ValueError("a request is prefilled once; decode continues it")
        T = int(ids.numel())
        if not 0 < T <= self.max_context:
            raise ValueError("the prompt does not fit the context")
        pages = self._allocate(T)
        table = torch.tensor(pages, device=ids.device)
        ids = ids.view(1, T)
        cos, sin = rope_tables(T, self.c.head_dim, self.c.rope_theta, ids.device)
        x = self.model.embed(ids)
        try:
            for i, blk in enumerate(self.model.layers):
                ve = self.model.value_embeds[str(i)](ids) if str(i) in self.model.value_embeds else None
                h = blk.input_norm(x)
                q, k1, k2, v1, v2 = blk.attn.operands(h, ve, cos, sin)
                self.caches[i].write(table, 0, k1[0], k2[0], v1[0], v2[0])
                x = x + blk.attn.reduce(h, q, k1, k2, v1, v2)
                x = x + blk.down(block_ops.swiglu(blk.gate_up(blk.post_norm(x))))
        except Exception:
            for cache in self.caches:
                cache.release(list(pages))
            raise
        self.requests[request] = _Request(T, pages)
        return self.model.lm_head(self.model.norm(x))[0, -1].float()

    @torch.inference_mode()
    def decode(self, requests: list[str], tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B] (one per request) -> logits [B, vocab] (fp32)."""
        rs = [self.requests[r] for r in requests]
        if len(set(requests)) != len(requests) or tokens.numel() != len(rs):
            raise ValueError("one token per distinct live request")
        dev = tokens.device
        for r in rs:                                                     # room for the new position, before anything is written
            if r.length + 1 > self.max_context:
                raise ValueError("a request reached the context limit")
            if r.length + 1 > len(r.pages) * PAGE:
                r.pages += self._allocate(1)
        B, c = len(rs), self.c
        position = torch.tensor([r.length for r in rs], device=dev)
        table = torch.zeros(B, self.max_pages, dtype=torch.int32, device=dev)
        for b, r in enumerate(rs):
            table[b, :len(r.pages)] = torch.tensor(r.pages, dtype=torch.int32, device=dev)
        seq_lens = (position + 1).int()
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=dev, dtype=torch.float32) / c.head_dim))
        ang = position.float()[:, None] * inv[None, :]
        x = self.model.embed(tokens.view(B, 1))
        for i, blk in enumerate(self.model.layers):
            ve = self.model.value_embeds[str(i)](tokens.view(B, 1)) if str(i) in self.model.value_embeds else None
            h = blk.input_norm(x)
            # every request sits at its own position: rotate row by row (B is small in decode)
            parts = [blk.attn.operands(h[b:b + 1], None if ve is None else ve[b:b + 1], ang[b:b + 1].cos(), ang[b:b + 1].sin()) for b in range(B)]
            q, k1, k2, v1, v2 = (torch.cat([p[j] for p in parts], 0) for j in range(5))
            cache = self.caches[i]
            for b, r in enumerate(rs):
                cache.write(table[b, :len(r.pages)].long(), r.length, k1[b], k2[b], v1[b], v2[b])
            w1, w2 = self._windows(blk.attn)
            y = simplicial_decode(q[:, 0], cache, table, seq_lens, w1, w2, blk.attn.conversion.scaling)
            x = x + blk.attn.native.finish(h, y.unsqueeze(1).to(h.dtype))
            x = x + blk.down(block_ops.swiglu(blk.gate_up(blk.post_norm(x))))
        for r in rs:
            r.length += 1
        return self.model.lm_head(self.model.norm(x))[:, -1].float()

    def free_pages(self) -> int:
        return len(self.caches[0].free)
