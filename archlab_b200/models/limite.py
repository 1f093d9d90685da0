"""Limite family: a gated-attention GQA decoder with sliding / global layers, and what the conversion and
agentic-RL experiments hang on it.

* ``LimiteLM``            - native decoder (fused QKV, per-head sigmoid output gate read from the first
                            ``attn_gate_channels`` of the hidden state, value embeddings on chosen layers,
                            SwiGLU, sliding-window layers with a few global ones).
* ``AttentionPrelude``    - trainable attention adapter in front of every block (zero-initialised output,
                            so installation leaves the function unchanged); ``set_trainable_mode`` switches
                            between training everything and training the adapters only.
* ``LimiteSimplicialAttention`` - conversion of a native attention into 2-simplicial attention that keeps
                            every native parameter: short keys / values are ``1 + delta(h)`` with a
                            zero-initialised delta, which makes the converted layer EQUAL the native one at
                            initialisation (a constant short factor cancels in the joint softmax).
* FLOP ledger             - closed-form causal pair / triple counts and per-token training FLOPs of the
                            native and converted model, and MFU against a stated peak.
* ``chunked_logits_processor`` - vocabulary projection + per-token processor over bounded sequence chunks
                            under activation checkpointing (no [sequence, vocabulary] buffer).
* ``StaticDecodeCache`` / ``GraphDecoder`` - fixed-address KV caches and a single-token decode step that is
                            captured once in a CUDA graph and replayed (eager on CPU).

Behavioural counterparts in the reference: src/archlab/architectures/limite_adapter.py:178-525,
limite_conversion.py:31-261, limite_cost.py:15-140, limite_head.py:12-55, limite_decode.py:20-230.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..ops import block_ops
from ..ops import simplicial as sx
from ..ops.attention import causal_attention
from .blocks import RMSNorm, apply_rope, rope_tables


@dataclass(frozen=True)
class LimiteConfig:
    vocab_size: int = 151_936
    hidden_size: int = 2048
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    num_key_value_heads: int = 4
    head_dim: int = 128
    intermediate_size: int = 6144
    sliding_window: int = 1023               # keys before the query that a local layer sees
    global_layers: tuple = (5, 11, 17, 23)
    ve_layers: tuple = (0, 12)
    attn_gate_channels: int = 12
    ve_gate_channels: int = 12
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    conversion: dict = field(default_factory=dict)      # {"short_window": w1} once converted

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(vocab_size=128, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                             head_dim=16, intermediate_size=128, sliding_window=7, global_layers=(3,), ve_layers=(0,)), **kw})

    @property
    def window_span(self) -> int:
        return self.sliding_window + 1


class LimiteAttention(nn.Module):
    def __init__(self, c: LimiteConfig, layer: int):
        super().__init__()
        self.c, self.layer_idx = c, layer
        self.is_global = layer in c.global_layers
        self.q_size, self.kv_size = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        self.qkv_proj = nn.Linear(c.hidden_size, self.q_size + 2 * self.kv_size, bias=False)
        self.o_proj = nn.Linear(self.q_size, c.hidden_size, bias=False)
        self.gate = nn.Linear(c.attn_gate_channels, c.num_attention_heads, bias=False)
        self.ve_gate = nn.Linear(c.ve_gate_channels, c.num_key_value_heads, bias=False) if layer in c.ve_layers else None
        self.q_norm, self.k_norm = RMSNorm(c.head_dim, c.rms_eps), RMSNorm(c.head_dim, c.rms_eps)

    def project(self, h, value_embeds, cos, sin):
        c = self.c
        B, T, _ = h.shape
        q, k, v = self.qkv_proj(h).split([self.q_size, self.kv_size, self.kv_size], -1)
        q = apply_rope(self.q_norm(q.view(B, T, c.num_attention_heads, c.head_dim)), cos, sin)
        k = apply_rope(self.k_norm(k.view(B, T, c.num_key_value_heads, c.head_dim)), cos, sin)
        v = v.view(B, T, c.num_key_value_heads, c.head_dim)
        if self.ve_gate is not None and value_embeds is not None:
            g = 2 * torch.sigmoid(self.ve_gate(h[..., : c.ve_gate_channels]))
            v = v + g.unsqueeze(-1) * value_embeds.view_as(v)
        return q, k, v

    def finish(self, h, y):
        g = torch.sigmoid(self.gate(h[..., : self.c.attn_gate_channels]))
        return self.o_proj((y * g.unsqueeze(-1).to(y.dtype)).flatten(-2))

    def reduce(self, q, k, v):
        return causal_attention(q, k, v, -1 if self.is_global else self.c.sliding_window)

    def forward(self, h, value_embeds, cos, sin):
        q, k, v = self.project(h, value_embeds, cos, sin)
        return self.finish(h, self.reduce(q, k, v))


class LimiteBlock(nn.Module):
    def __init__(self, c: LimiteConfig, layer: int):
        super().__init__()
        self.input_norm, self.post_norm = RMSNorm(c.hidden_size, c.rms_eps), RMSNorm(c.hidden_size, c.rms_eps)
        self.attn = LimiteAttention(c, layer)
        self.gate_up = nn.Linear(c.hidden_size, 2 * c.intermediate_size, bias=False)
        self.down = nn.Linear(c.intermediate_size, c.hidden_size, bias=False)
        self.prelude = None

    def forward(self, x, ve, cos, sin):
        if self.prelude is not None:
            x = x + self.prelude(x, cos, sin)
        x = x + self.attn(self.input_norm(x), ve, cos, sin)
        return x + self.down(block_ops.swiglu(self.gate_up(self.post_norm(x))))


class LimiteLM(nn.Module):
    def __init__(self, config: LimiteConfig):
        super().__init__()
        c = self.config = config
        self.embed = nn.Embedding(c.vocab_size, c.hidden_size)
        self.value_embeds = nn.ModuleDict({str(i): nn.Embedding(c.vocab_size, c.num_key_value_heads * c.head_dim) for i in c.ve_layers})
        self.layers = nn.ModuleList(LimiteBlock(c, i) for i in range(c.num_hidden_layers))
        self.norm = RMSNorm(c.hidden_size, c.rms_eps)
        self.lm_head = nn.Linear(c.hidden_size, c.vocab_size, bias=False)

    def init_weights(self, std: float = 0.02):
        for p in self.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, std=std)

    def hidden(self, ids):
        c = self.config
        cos, sin = rope_tables(ids.size(1), c.head_dim, c.rope_theta, ids.device)
        x = self.embed(ids)
        for i, blk in enumerate(self.layers):
            ve = self.value_embeds[str(i)](ids) if str(i) in self.value_embeds else None
            x = blk(x, ve, cos, sin)
        return self.norm(x)

    def forward(self, ids, labels=None):
        logits = self.lm_head(self.hidden(ids))
        if labels is None:
            return logits.float()
        flat = labels.flatten()
        return block_ops.cross_entropy_sum(logits.flatten(0, 1), flat) / flat.ne(-1).sum().clamp_min(1)


# ------------------------------------------------------------------------------------------------
# adapters
# ------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class AdapterConfig:
    heads: int = 4
    head_dim: int = 32
    window: int = 255


class AttentionPrelude(nn.Module):
    """Small windowed attention read of the residual stream, added before the block; output zero-initialised."""

    def __init__(self, c: LimiteConfig, a: AdapterConfig):
        super().__init__()
        self.a = a
        self.norm = RMSNorm(c.hidden_size, c.rms_eps)
        self.qkv = nn.Linear(c.hidden_size, 3 * a.heads * a.head_dim, bias=False)
        self.out = nn.Linear(a.heads * a.head_dim, c.hidden_size, bias=False)
        nn.init.zeros_(self.out.weight)

    def forward(self, x, cos, sin):
        a = self.a
        B, T, _ = x.shape
        q, k, v = (t.view(B, T, a.heads, a.head_dim) for t in self.qkv(self.norm(x)).chunk(3, -1))
        r = min(a.head_dim, 2 * cos.size(-1))
        q, k = apply_rope(q, cos[:, : r // 2], sin[:, : r // 2], rot_dim=r), apply_rope(k, cos[:, : r // 2], sin[:, : r // 2], rot_dim=r)
        return self.out(causal_attention(q, k, v, a.window).flatten(-2))


def install_adapters(model: LimiteLM, a: AdapterConfig) -> LimiteLM:
    for blk in model.layers:
        if blk.prelude is not None:
            raise ValueError("adapters are already installed")
        blk.prelude = AttentionPrelude(model.config, a).to(next(model.parameters()).device)
    return model


def adapter_state(model) -> dict:
    return {k: v for k, v in model.state_dict().items() if ".prelude." in k}


def backbone_state(model) -> dict:
    return {k: v for k, v in model.state_dict().items() if ".prelude." not in k}


def set_trainable_mode(model, mode: str) -> int:
    """``full``: every parameter trains; ``adapter``: only the preludes.  Returns the trainable count."""
    if mode not in ("full", "adapter"):
        raise ValueError("trainable mode is full or adapter")
    n = 0
    for name, p in model.named_parameters():
        p.requires_grad_(mode == "full" or ".prelude." in name)
        n += p.numel() if p.requires_grad else 0
    return n


# ------------------------------------------------------------------------------------------------
# conversion to 2-simplicial attention
# ------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class ConversionConfig:
    short_window: int = 8
    # Which implementation reduces the converted layers (the reference's conversion.backend tri-state,
    # src/archlab/architectures/limite_conversion.py:65-120):
    #   "auto"       sm_100a kernel when dtype / head width allow, else the PyTorch statement
    #   "kernel"     the sm_100a kernel or an error (a run that must not silently fall back)
    #   "reference"  the PyTorch statement with fp32 queries (oracle runs)
    backend: str = "auto"
    scaling: float | None = None              # softmax scale of the reduction; None = head_dim ** -0.5

    def __post_init__(self):
        if self.backend not in ("auto", "kernel", "reference"):
            raise ValueError(f"unknown conversion backend {self.backend!r}")


def query_for_fixed_scale(q: torch.Tensor, scaling: float, kernel_scale: float) -> torch.Tensor:
    """A reduction backend that hard-codes its own softmax scale (the reference's packed kernels apply D ** -0.5)
    still realises the model's ``scaling`` when the query is multiplied by ``scaling / kernel_scale`` first, in
    fp32 (fp64 stays fp64) so that the factor is not rounded into the bf16 query."""
    work = torch.float64 if q.dtype == torch.float64 else torch.float32
    return q.to(work) * (scaling / kernel_scale)


class LimiteSimplicialAttention(nn.Module):
    """Keeps the native module (projections, norms, gates) and replaces only the reduction by the joint
    softmax over (short key, long key) pairs with k1 = 1 + dK(h), v1 = 1 + dV(h)."""

    def __init__(self, native: LimiteAttention, config: ConversionConfig):
        super().__init__()
        self.native, self.conversion = native, config
        w = native.qkv_proj.weight
        self.short_kv_delta = nn.Parameter(w.new_zeros(2 * native.kv_size, w.shape[1]))

    def operands(self, h, value_embeds, cos, sin):
        """(q, k1, k2, v1, v2) of the tokens in ``h``; serving caches k1 / v1 (short) and k2 / v2 (long) per layer."""
        n, c = self.native, self.native.c
        q, k2, v2 = n.project(h, value_embeds, cos, sin)
        B, T = h.shape[:2]
        dk, dv = F.linear(h, self.short_kv_delta.to(h.dtype)).split(n.kv_size, -1)
        k1 = 1 + dk.view(B, T, c.num_key_value_heads, c.head_dim)
        v1 = 1 + dv.view(B, T, c.num_key_value_heads, c.head_dim)
        return q, k1, k2, v1, v2

    def forward(self, h, value_embeds, cos, sin):
        return self.reduce(h, *self.operands(h, value_embeds, cos, sin))

    def reduce(self, h, q, k1, k2, v1, v2):
        n, c = self.native, self.native.c
        T = h.shape[1]
        w2 = T if n.is_global else c.window_span
        w1 = min(self.conversion.short_window, w2)
        scaling, backend = self.conversion.scaling, self.conversion.backend
        if backend == "reference":
            y = sx.simplicial_attention_reference(q.float(), k1.float(), k2.float(), v1.float(), v2.float(), w1, w2, scale=scaling)
        else:
            if backend == "kernel":
                from ..ops.simplicial_cuda import kernel_supports

                if not (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and kernel_supports(q, k1, v1, w1, w2)):
                    raise RuntimeError("conversion.backend = 'kernel' but the sm_100a simplicial kernel does not take this "
                                       f"input (device {q.device}, dtype {q.dtype}, head_dim {q.shape[-1]}, windows {w1} x {w2})")
            y = sx.simplicial_attention(q, k1.to(q.dtype), k2, v1.to(q.dtype), v2, w1, w2, scale=scaling)
        return n.finish(h, y.to(h.dtype))


def replace_limite_attention(model: LimiteLM, config: ConversionConfig) -> LimiteLM:
    for blk in model.layers:
        if isinstance(blk.attn, LimiteSimplicialAttention):
            raise ValueError("model is already converted")
        blk.attn = LimiteSimplicialAttention(blk.attn, config)
    object.__setattr__(model.config, "conversion", {"short_window": config.short_window})
    return model


def conversion_metadata(model) -> dict:
    conv = [b.attn for b in model.layers if isinstance(b.attn, LimiteSimplicialAttention)]
    return {"converted_layers": len(conv), "short_window": conv[0].conversion.short_window if conv else None,
            "new_parameters": sum(a.short_kv_delta.numel() for a in conv)}


# ------------------------------------------------------------------------------------------------
# FLOP ledger
# ------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class FlopLedger:
    linear_per_token: int
    attention_per_token: float
    sequence_length: int

    @property
    def per_token(self) -> float:
        return self.linear_per_token + self.attention_per_token

    def mfu(self, tokens: int, seconds: float, world_size: int, peak: float = 2.25e15) -> float:
        if tokens < 0 or seconds <= 0 or world_size < 1 or peak <= 0:
            raise ValueError("invalid MFU measurement")
        return tokens * self.per_token / (seconds * world_size * peak)


def causal_pairs(length: int, span: int | None = None) -> int:
    """Number of (query, key) pairs with key <= query (and key > query - span)."""
    if length < 1 or (span is not None and span < 1):
        raise ValueError("length and span must be positive")
    w = min(length, span) if span is not None else length
    return w * (w + 1) // 2 + (length - w) * w


def causal_triples(length: int, short_span: int, long_span: int) -> int:
    """Sum over queries i of min(i+1, a) * min(i+1, b), in closed form."""
    causal_pairs(length, short_span)
    causal_pairs(length, long_span)
    a, b = sorted((min(length, short_span), min(length, long_span)))
    return a * (a + 1) * (2 * a + 1) // 6 + a * (b * (b + 1) - a * (a + 1)) // 2 + (length - b) * a * b


def _attention_matrix_coefficients(c: LimiteConfig) -> int:
    return (c.num_hidden_layers * c.hidden_size * c.head_dim * (2 * c.num_attention_heads + 2 * c.num_key_value_heads)
            + c.num_hidden_layers * c.num_attention_heads * c.attn_gate_channels
            + len(set(c.ve_layers)) * c.num_key_value_heads * c.ve_gate_channels)


def baseline_flops(c: LimiteConfig, sequence_length: int, trainable_mode: str = "full") -> FlopLedger:
    """Training FLOPs per token: 6 per trained coefficient, 4 per frozen one that still back-propagates
    activations (adapter mode), plus 12 * heads * head_dim per causal (query, key) pair."""
    if trainable_mode not in ("full", "adapter"):
        raise ValueError("unsupported trainable mode")
    L = sequence_length
    if any(i < 0 or i >= c.num_hidden_layers for i in c.global_layers):
        raise ValueError("invalid global layer indices")
    attn = _attention_matrix_coefficients(c)
    mlp = c.num_hidden_layers * 3 * c.hidden_size * c.intermediate_size
    head = c.vocab_size * c.hidden_size
    per = 6 if trainable_mode == "full" else 4
    linear = per * (attn + mlp + head)
    g = len(set(c.global_layers))
    pairs = g * causal_pairs(L) + (c.num_hidden_layers - g) * causal_pairs(L, c.window_span)
    return FlopLedger(linear, 12 * c.num_attention_heads * c.head_dim * pairs / L, L)


def converted_flops(c: LimiteConfig, sequence_length: int) -> FlopLedger:
    """As above with every attention replaced: the short projection's coefficients are added, and the
    reductions count causal (query, short key, long key) triples."""
    if not c.conversion:
        raise ValueError("the configuration is not converted")
    L, base = sequence_length, baseline_flops(c, sequence_length, "full")
    short_proj = c.num_hidden_layers * c.hidden_size * c.head_dim * 2 * c.num_key_value_heads
    w1, g = c.conversion["short_window"], len(set(c.global_layers))
    triples = g * causal_triples(L, w1, L) + (c.num_hidden_layers - g) * causal_triples(L, min(w1, c.window_span), c.window_span)
    return FlopLedger(base.linear_per_token + 6 * short_proj, 12 * c.num_attention_heads * c.head_dim * triples / L, L)


# ------------------------------------------------------------------------------------------------
# chunked head
# ------------------------------------------------------------------------------------------------
def chunked_logits_processor(head, hidden, processor, processor_args: dict, *, chunk_size: int = 512) -> dict:
    """``processor(logits, **args) -> {name: [B, t, ...]}`` applied to ``head(hidden)`` over sequence chunks;
    chunks are re-computed in backward (non-reentrant checkpointing), so only one chunk of logits lives
    at a time."""
    if hidden.ndim != 3 or hidden.shape[1] == 0 or type(chunk_size) is not int or chunk_size < 1:
        raise ValueError("invalid head chunk geometry")
    names, values = tuple(processor_args), tuple(processor_args.values())
    if not values or any(not isinstance(v, torch.Tensor) or v.shape[:2] != hidden.shape[:2] for v in values):
        raise ValueError("processor arguments must be [batch, sequence, ...] tensors")

    def part(x, *args):
        return processor(head(x), **{n: a.clone() for n, a in zip(names, args)})

    chunks = []
    for s in range(0, hidden.shape[1], chunk_size):
        args = (hidden[:, s:s + chunk_size], *(v[:, s:s + chunk_size] for v in values))
        res = checkpoint(part, *args, use_reentrant=False) if torch.is_grad_enabled() else part(*args)
        if not isinstance(res, dict) or not res or any(v.shape[:2] != args[0].shape[:2] for v in res.values()):
            raise ValueError("the processor must return per-token tensors")
        chunks.append(res)
    if any(ch.keys() != chunks[0].keys() for ch in chunks):
        raise ValueError("processor outputs differ between chunks")
    return {n: torch.cat([ch[n] for ch in chunks], 1) for n in chunks[0]}


def logprob_entropy_processor(logits, labels, temperature=None):
    lf = logits.float()
    if temperature is not None:
        lf = lf / temperature.unsqueeze(-1)
    lp = F.log_softmax(lf, -1)
    return {"log_probs": lp.gather(-1, labels.unsqueeze(-1)).squeeze(-1), "entropy": -(lp.exp() * lp).sum(-1)}


# ------------------------------------------------------------------------------------------------
# static caches and graph decoding
# ------------------------------------------------------------------------------------------------
class StaticDecodeCache:
    """Per-layer K/V buffers of fixed capacity (local layers keep a ring of ``window_span`` rows); the current
    position lives in a device tensor so that a captured graph reads it at replay time."""

    def __init__(self, c: LimiteConfig, batch: int, capacity: int, device, dtype):
        self.c, self.capacity = c, capacity
        self.sizes = [capacity if i in c.global_layers else min(capacity, c.window_span) for i in range(c.num_hidden_layers)]
        mk = lambda n: torch.zeros(batch, n, c.num_key_value_heads, c.head_dim, device=device, dtype=dtype)
        self.k, self.v = [mk(n) for n in self.sizes], [mk(n) for n in self.sizes]
        self.position = torch.zeros(1, dtype=torch.long, device=device)

    @torch.no_grad()
    def load_prefill(self, ks, vs) -> None:
        T = ks[0].size(1)
        if T > self.capacity:
            raise ValueError("prefill exceeds the cache capacity")
        for i, n in enumerate(self.sizes):
            self.k[i].zero_(), self.v[i].zero_()
            pos = torch.arange(max(0, T - n), T, device=ks[i].device)
            self.k[i][:, pos % n] = ks[i][:, pos]
            self.v[i][:, pos % n] = vs[i][:, pos]
        self.position.fill_(T)

    def write(self, layer: int, k, v) -> None:
        slot = (self.position % self.sizes[layer]).view(1, 1, 1, 1).expand(k.size(0), 1, *k.shape[2:])
        self.k[layer].scatter_(1, slot, k)
        self.v[layer].scatter_(1, slot, v)

    def valid_mask(self, layer: int):
        """[n] bool: slots that hold a key visible to the token at ``position`` (after it has been written)."""
        n = self.sizes[layer]
        return torch.arange(n, device=self.position.device) < torch.clamp(self.position + 1, max=n)


@torch.no_grad()
def prefill(model: LimiteLM, ids):
    """Full forward that also returns the per-layer keys / values for the cache."""
    c = model.config
    cos, sin = rope_tables(ids.size(1), c.head_dim, c.rope_theta, ids.device)
    x, ks, vs = model.embed(ids), [], []
    for i, blk in enumerate(model.layers):
        ve = model.value_embeds[str(i)](ids) if str(i) in model.value_embeds else None
        if blk.prelude is not None:
            x = x + blk.prelude(x, cos, sin)
        h = blk.input_norm(x)
        q, k, v = blk.attn.project(h, ve, cos, sin)
        ks.append(k), vs.append(v)
        x = x + blk.attn.finish(h, blk.attn.reduce(q, k, v))
        x = x + blk.down(block_ops.swiglu(blk.gate_up(blk.post_norm(x))))
    return model.lm_head(model.norm(x))[:, -1].float(), ks, vs


def decode_step(model: LimiteLM, cache: StaticDecodeCache, token):
    """One token through the model against the static cache; no data-dependent shapes or host reads."""
    c = model.config
    inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=token.device, dtype=torch.float32) / c.head_dim))
    ang = cache.position.float()[:, None] * inv[None, :]
    cos, sin = ang.cos(), ang.sin()
    x = model.embed(token)
    rep = c.num_attention_heads // c.num_key_value_heads
    for i, blk in enumerate(model.layers):
        if blk.prelude is not None:
            raise ValueError("static decoding covers the native backbone")
        ve = model.value_embeds[str(i)](token) if str(i) in model.value_embeds else None
        h = blk.input_norm(x)
        q, k, v = blk.attn.project(h, ve, cos, sin)
        cache.write(i, k, v)
        kk, vv = cache.k[i].repeat_interleave(rep, 2), cache.v[i].repeat_interleave(rep, 2)
        s = torch.einsum("bqhd,bshd->bhqs", q.float(), kk.float()) * c.head_dim ** -0.5
        s = s.masked_fill(~cache.valid_mask(i).view(1, 1, 1, -1), float("-inf"))
        y = torch.einsum("bhqs,bshd->bqhd", s.softmax(-1), vv.float()).to(x.dtype)
        x = x + blk.attn.finish(h, y)
        x = x + blk.down(block_ops.swiglu(blk.gate_up(blk.post_norm(x))))
    cache.position += 1
    return model.lm_head(model.norm(x))[:, -1].float()


class GraphDecoder:
    """Owns the static cache and input buffers; on CUDA the decode step is captured once and replayed."""

    def __init__(self, model: LimiteLM, batch: int, capacity: int, *, capture: bool | None = None):
        if model.training or torch.is_grad_enabled():
            raise ValueError("graph decoding needs eval mode under no_grad")
        p = next(model.parameters())
        self.model = model
        self.cache = StaticDecodeCache(model.config, batch, capacity, p.device, p.dtype)
        self.token = torch.zeros(batch, 1, dtype=torch.long, device=p.device)
        self.graph, self.logits = None, None
        self.capture = p.is_cuda if capture is None else capture

    def reset(self, ks, vs, first_token) -> None:
        self.cache.load_prefill(ks, vs)
        self.token.copy_(first_token)
        if self.capture and self.graph is None:
            saved = [t.clone() for t in (*self.cache.k, *self.cache.v, self.cache.position)]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):                           # warm library workspaces outside the capture
                    decode_step(self.model, self.cache, self.token)
            torch.cuda.current_stream().wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.logits = decode_step(self.model, self.cache, self.token)
            for dst, src in zip((*self.cache.k, *self.cache.v, self.cache.position), saved):
                dst.copy_(src)

    def __call__(self, token):
        if int(self.cache.position) >= self.cache.capacity:
            raise ValueError("decode position exceeds the preallocated context")
        self.token.copy_(token)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.logits = decode_step(self.model, self.cache, self.token)
        return self.logits


class GraphDecoderPool:
    """One decoder per (batch, capacity) geometry, reused across requests."""

    def __init__(self, model):
        self.model, self.pool = model, {}

    def get(self, batch: int, capacity: int) -> GraphDecoder:
        key = (batch, capacity)
        if key not in self.pool:
            self.pool[key] = GraphDecoder(self.model, batch, capacity)
        return self.pool[key]


from .protocol import attach_protocol  # noqa: E402  (after the classes it completes)

attach_protocol(LimiteLM)
