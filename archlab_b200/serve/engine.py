"""Continuous-batching generation engine for Limite models converted to 2-simplicial attention.

Every layer owns four paged caches (short keys / values ``1 + delta(h)``, long keys / values) carved
into 128-position pages; a request holds a page list per engine (the same logical page index maps to
the same physical page in every layer, so one block table serves all layers).  ``step()`` admits waiting
requests (prefill: one full forward through the training kernels that also fills the pages) and then
advances ALL running sequences by one token in one batched pass - per layer one projection GEMM, one
cache write and one launch of the paged decode mode of the tcgen05 simplicial kernel.  Finished requests
release their pages at once.

Stands where the reference bridges into vLLM (src/archlab/training/serving.py, serving_conversion.py:
a model class with two cache owners per layer, prefill through the training kernel, decode over
gathered cache windows); here the scheduler, the page allocator and the kernels are the framework's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..models import limite as L
from ..models.blocks import rope_tables
from ..ops import block_ops
from ..ops.simplicial_decode import PAGE, PagedSimplicialCache, simplicial_decode


@dataclass
class Request:
    rid: int
    prompt: list[int]
    max_new_tokens: int
    eos: int | None = None
    pages: list[int] = field(default_factory=list)
    tokens: list[int] = field(default_factory=list)       # generated so far
    length: int = 0                                       # positions in the cache

    @property
    def done(self) -> bool:
        return len(self.tokens) >= self.max_new_tokens or (self.eos is not None and self.tokens and self.tokens[-1] == self.eos)


@dataclass(frozen=True)
class ServingSettings:
    """What a deployment asks of the engine; ``validate_serving`` refuses what the paged simplicial path does not implement."""
    tensor_parallel: int = 1
    pipeline_parallel: int = 1
    chunked_prefill: bool = False
    prefix_caching: bool = False
    cache_dtype: str = "auto"
    speculative: bool = False
    quantization: str | None = None


def validate_serving(model: L.LimiteLM, settings: ServingSettings, *, short_window: int | None = None) -> None:
    """The engine prefills one COMPLETE prompt per request and owns private, unquantised pages per request: tensor /
    pipeline splits, chunked prefill, prefix sharing, quantised caches or weights and speculative decoding are refused
    rather than silently ignored, and so is a model that is not converted in every layer or still carries adapters
    (the reference states the same admission rules for its engine bridge: src/archlab/training/serving_conversion.py:19-46)."""
    if settings.tensor_parallel != 1 or settings.pipeline_parallel != 1:
        raise ValueError("converted serving runs on one GPU per replica (TP = PP = 1)")
    if settings.chunked_prefill:
        raise ValueError("converted serving admits one complete prompt at a time (no chunked prefill)")
    if settings.prefix_caching or settings.cache_dtype not in ("auto", "bfloat16", "float16", "float32"):
        raise ValueError("converted serving needs private, unquantised K/V pages")
    if settings.quantization is not None or settings.speculative:
        raise ValueError("converted serving does not admit quantisation or speculative decoding")
    layers = [b.attn for b in model.layers]
    if not all(isinstance(a, L.LimiteSimplicialAttention) for a in layers) or any(b.prelude is not None for b in model.layers):
        raise ValueError("converted serving needs the attention replacement in every layer and no adapters")
    if short_window is not None and any(a.conversion.short_window != short_window for a in layers):
        raise ValueError(f"converted serving was qualified for short window {short_window}")


class SimplicialServingEngine:
    def __init__(self, model: L.LimiteLM, *, num_pages: int, max_batch: int = 64, max_seq_len: int = 4096, settings: ServingSettings | None = None):
        if settings is not None:
            validate_serving(model, settings)
        if not all(isinstance(b.attn, L.LimiteSimplicialAttention) for b in model.layers):
            raise ValueError("the engine serves models whose attention layers were converted")
        if any(b.prelude is not None for b in model.layers):
            raise ValueError("adapters are a training-time construct")
        self.model = model.eval()
        c = self.c = model.config
        p = next(model.parameters())
        self.device, self.dtype = p.device, p.dtype
        self.caches = [PagedSimplicialCache(num_pages, c.num_key_value_heads, c.head_dim, p.device, p.dtype) for _ in model.layers]
        self.free = list(range(num_pages - 1, -1, -1))
        self.max_batch, self.max_pages = max_batch, (max_seq_len + PAGE - 1) // PAGE
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self.finished: dict[int, list[int]] = {}
        self._next = 0
        self.w1 = model.layers[0].attn.conversion.short_window

    # -- requests ------------------------------------------------------------------------------------
    def add_request(self, prompt: list[int], max_new_tokens: int, eos: int | None = None) -> int:
        if not prompt or len(prompt) + max_new_tokens > self.max_pages * PAGE:
            raise ValueError("empty prompt or request longer than the engine's sequence limit")
        self._next += 1
        self.waiting.append(Request(self._next, list(prompt), max_new_tokens, eos))
        return self._next

    def _pages_for(self, n: int) -> int:
        return (n + PAGE - 1) // PAGE

    def _grow(self, r: Request, length: int) -> bool:
        need = self._pages_for(length) - len(r.pages)
        if need > len(self.free):
            return False
        r.pages += [self.free.pop() for _ in range(need)]
        return True

    def _release(self, r: Request) -> None:
        self.free.extend(r.pages)
        r.pages = []

    # -- model pieces --------------------------------------------------------------------------------
    def _layer_window(self, attn: L.LimiteSimplicialAttention) -> int:
        return self.max_pages * PAGE if attn.native.is_global else self.c.window_span

    def _short(self, attn, h):
        n = attn.native
        dk, dv = torch.nn.functional.linear(h, attn.short_kv_delta.to(h.dtype)).split(n.kv_size, -1)
        shape = (*h.shape[:2], self.c.num_key_value_heads, self.c.head_dim)
        return 1 + dk.view(shape), 1 + dv.view(shape)

    @torch.no_grad()
    def _prefill(self, r: Request) -> int:
        m, c = self.model, self.c
        ids = torch.tensor([r.prompt], device=self.device)
        T = ids.size(1)
        pages = torch.tensor(r.pages, device=self.device)
        cos, sin = rope_tables(T, c.head_dim, c.rope_theta, self.device)
        x = m.embed(ids)
        for i, blk in enumerate(m.layers):
            ve = m.value_embeds[str(i)](ids) if str(i) in m.value_embeds else None
            h = blk.input_norm(x)
            q, k2, v2 = blk.attn.native.project(h, ve, cos, sin)
            k1, v1 = self._short(blk.attn, h)
            self.caches[i].write(pages, 0, k1[0], k2[0], v1[0], v2[0])
            x = x + blk.attn(h, ve, cos, sin)                  # the training forward (same projections, fused kernel)
            x = x + blk.down(block_ops.swiglu(blk.gate_up(blk.post_norm(x))))
        r.length = T
        return int(m.lm_head(m.norm(x))[0, -1].float().argmax())

    @torch.no_grad()
    def _decode(self, batch: list[Request]) -> list[int]:
        m, c = self.model, self.c
        B = len(batch)
        tok = torch.tensor([[r.tokens[-1]] for r in batch], device=self.device)
        pos = torch.tensor([r.length for r in batch], device=self.device)                 # position of the new token
        table = torch.zeros(B, self.max_pages, dtype=torch.int32, device=self.device)
        for b, r in enumerate(batch):
            table[b, : len(r.pages)] = torch.tensor(r.pages, dtype=torch.int32, device=self.device)
        rows = table.gather(1, (pos // PAGE).view(B, 1).long()).view(B).long() * PAGE + pos % PAGE
        seq_lens = (pos + 1).int()
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=self.device, dtype=torch.float32) / c.head_dim))
        ang = pos.float()[:, None] * inv[None, :]
        x = m.embed(tok)
        for i, blk in enumerate(m.layers):
            ve = m.value_embeds[str(i)](tok) if str(i) in m.value_embeds else None
            h = blk.input_norm(x)
            # per-sequence rotary angle: treat the batch as the "time" axis of a [1, B, H, D] tensor
            q, k2, v2 = blk.attn.native.project(h.transpose(0, 1), None if ve is None else ve.transpose(0, 1), ang.cos(), ang.sin())
            k1, v1 = self._short(blk.attn, h.transpose(0, 1))
            cache = self.caches[i]
            for dst, src in ((cache.k1, k1), (cache.k2, k2), (cache.v1, v1), (cache.v2, v2)):
                dst[rows] = src[0].reshape(B, -1).to(dst.dtype)
            w2 = self._layer_window(blk.attn)
            y = simplicial_decode(q[0].contiguous(), cache, table, seq_lens, min(self.w1, w2), w2)
            x = x + blk.attn.native.finish(h, y.unsqueeze(1).to(h.dtype))
            x = x + blk.down(block_ops.swiglu(blk.gate_up(blk.post_norm(x))))
        for r in batch:
            r.length += 1
        return m.lm_head(m.norm(x))[:, -1].float().argmax(-1).tolist()

    # -- scheduler -----------------------------------------------------------------------------------
    def step(self) -> dict:
        """Admit what fits, then advance every running sequence by one token."""
        admitted = 0
        while self.waiting and len(self.running) < self.max_batch:
            r = self.waiting[0]
            if not self._grow(r, len(r.prompt) + 1):
                break                                          # wait for pages to come back
            self.waiting.pop(0)
            r.tokens.append(self._prefill(r))
            self.running.append(r)
            admitted += 1
        batch = [r for r in self.running if not r.done]
        stalled = [r for r in batch if not self._grow(r, r.length + 1)]
        for r in stalled:                                      # out of pages: preempt the newest, recompute later
            batch.remove(r)
            self.running.remove(r)
            self._release(r)
            self.waiting.insert(0, Request(r.rid, r.prompt + r.tokens, r.max_new_tokens - len(r.tokens), r.eos))
            self.finished.setdefault(-r.rid, []).extend(r.tokens)       # tokens already produced by the preempted run
        if batch:
            for r, t in zip(batch, self._decode(batch)):
                r.tokens.append(t)
        for r in [r for r in self.running if r.done]:
            self.running.remove(r)
            self._release(r)
            self.finished[r.rid] = self.finished.pop(-r.rid, []) + r.tokens
        return {"admitted": admitted, "decoded": len(batch), "running": len(self.running), "waiting": len(self.waiting),
                "free_pages": len(self.free)}

    def run_until_done(self, max_steps: int = 100000) -> dict[int, list[int]]:
        for _ in range(max_steps):
            if not self.waiting and not self.running:
                break
            self.step()
        return {k: v for k, v in self.finished.items() if k > 0}
