"""Kimi-style linear-attention language model: KDA (Kimi delta attention) token mixers in a
``KKKG`` pattern with NoPE gated global attention layers, and block attention-residual (AttnRes)
depth-wise reads.

KDA layer: q/k/v projections -> short depthwise causal conv + SiLU -> per-channel log-decay
``g = -exp(A_log) softplus(f_up(f_down x) + dt_bias)`` (variant ``kimi_k3``: ``-5 sigmoid``),
``beta = sigmoid`` (variant ``solar_negative``: ``2 sigmoid``, which lets the state map have
negative eigenvalues) -> delta rule, chunk 64 -> per-head RMSNorm * sigmoid(output gate) -> o_proj
(src/archlab/architectures/kimi.py:40-321; recurrence oracle :154-178; AttnRes :619-670).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.attention import causal_attention
from ..ops import delta_rule
from .blocks import rms_norm

KDA_PATTERN = "KKKG"
KDA_VARIANTS = ("kimi_linear", "kimi_k3", "solar_negative")


@dataclass
class KimiConfig:
    vocab_size: int = 32768
    sequence_len: int = 2048
    n_layer: int = 12
    n_head: int = 6
    n_embd: int = 768
    kda_pattern: str = KDA_PATTERN
    kda_chunk_size: int = 64
    kda_conv_size: int = 4
    kda_variant: str = "kimi_linear"
    kda_force_final_global: bool = True
    attnres_block: int = 0          # > 0: AttnRes read over block summaries every this many layers
    attnres_heads: int = 1
    softcap: float = 15.0

    def __post_init__(self):
        if self.kda_variant not in KDA_VARIANTS:
            raise ValueError(f"unknown kda_variant={self.kda_variant!r}")
        if self.n_embd % self.n_head:
            raise ValueError("n_embd must divide into heads")


def is_kda_layer(layer_idx: int, n_layer: int, pattern: str = KDA_PATTERN, force_final_global: bool = True) -> bool:
    if force_final_global and layer_idx == n_layer - 1:
        return False
    ch = pattern[layer_idx % len(pattern)].upper()
    if ch not in "KG":
        raise ValueError(f"Invalid KDA pattern {pattern!r}; use K and G only")
    return ch == "K"


def kda_layer_map(n_layer: int, pattern: str = KDA_PATTERN, force_final_global: bool = True) -> dict[str, list[int]]:
    kda = [i + 1 for i in range(n_layer) if is_kda_layer(i, n_layer, pattern, force_final_global)]
    return {"kda": kda, "global": [i + 1 for i in range(n_layer) if i + 1 not in kda]}


def _lin(i, o, bias=False):
    return nn.Linear(i, o, bias=bias)


class KimiDeltaAttention(nn.Module):
    def __init__(self, c: KimiConfig):
        super().__init__()
        self.h, self.d, self.variant, self.chunk = c.n_head, c.n_embd // c.n_head, c.kda_variant, c.kda_chunk_size
        E = c.n_embd
        self.q_proj, self.k_proj, self.v_proj = _lin(E, E), _lin(E, E), _lin(E, E)
        self.q_conv = nn.Parameter(torch.empty(E, c.kda_conv_size))
        self.k_conv = nn.Parameter(torch.empty(E, c.kda_conv_size))
        self.v_conv = nn.Parameter(torch.empty(E, c.kda_conv_size))
        self.f_down, self.f_up = _lin(E, self.d), _lin(self.d, E)
        self.beta_proj = _lin(E, self.h)
        self.a_log = nn.Parameter(torch.zeros(self.h))
        self.dt_bias = nn.Parameter(torch.zeros(E))
        if self.variant in ("kimi_k3", "solar_negative"):
            self.g_proj = _lin(E, E, bias=True)
        else:
            self.g_down, self.g_up = _lin(E, self.d), _lin(self.d, E, bias=True)
        self.output_norm_weight = nn.Parameter(torch.ones(self.d))
        self.o_proj = _lin(E, E)

    def gate(self, raw: torch.Tensor) -> torch.Tensor:
        """Per-channel log-decay [B, T, H, D] (<= 0)."""
        shaped = (raw.float() + self.dt_bias.float()).unflatten(-1, (self.h, self.d))
        a = self.a_log.float().exp().view(1, 1, self.h, 1)
        if self.variant == "kimi_k3":
            return -5.0 * torch.sigmoid(a * shaped)
        return -a * F.softplus(shaped)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, E = x.shape
        conv = lambda proj, w: delta_rule.causal_conv1d(proj(x), w).view(B, T, self.h, self.d)
        q, k, v = conv(self.q_proj, self.q_conv), conv(self.k_proj, self.k_conv), conv(self.v_proj, self.v_conv)
        g = self.gate(self.f_up(self.f_down(x)))
        beta = torch.sigmoid(self.beta_proj(x))
        if self.variant == "solar_negative":
            beta = 2.0 * beta
        y = delta_rule.chunk_kda(q, k, v, g, beta, chunk=self.chunk).to(x.dtype)
        og = self.g_proj(x) if hasattr(self, "g_proj") else self.g_up(self.g_down(x))
        y = rms_norm(y, self.output_norm_weight, eps=1e-5) * torch.sigmoid(og.view(B, T, self.h, self.d))
        return self.o_proj(y.reshape(B, T, E))


class GlobalGatedAttention(nn.Module):
    """Causal softmax attention with no positional encoding and a sigmoid output gate."""

    def __init__(self, c: KimiConfig):
        super().__init__()
        self.h, self.d = c.n_head, c.n_embd // c.n_head
        E = c.n_embd
        self.qkv = _lin(E, 3 * E)
        self.gate = _lin(E, E)
        self.o_proj = _lin(E, E)

    def forward(self, x):
        B, T, E = x.shape
        q, k, v = self.qkv(x).view(B, T, 3, self.h, self.d).unbind(2)
        q, k = rms_norm(q), rms_norm(k)
        o = causal_attention(q, k, v)
        return self.o_proj(o.reshape(B, T, E) * torch.sigmoid(self.gate(x)))


class AttnResRead(nn.Module):
    """One learned pseudo-query attends over residual sources (block summaries): softmax over the
    sources of ``(rmsnorm(source) * norm_weight) . query`` (per head), fp32 scores and sums."""

    def __init__(self, width: int, heads: int = 1, eps: float = 1e-6):
        super().__init__()
        if heads <= 0 or width % heads:
            raise ValueError("AttnRes width must be divisible by a positive head count")
        self.heads, self.eps = heads, eps
        self.query = nn.Parameter(torch.zeros(width))
        self.norm_weight = nn.Parameter(torch.ones(width))

    def forward(self, *sources: torch.Tensor) -> torch.Tensor:
        if not sources:
            raise ValueError("AttnRes requires at least one residual source")
        shape = sources[0].shape
        if any(s.shape != shape for s in sources):
            raise ValueError("all AttnRes sources must share a shape")
        hd = shape[-1] // self.heads
        w = (self.norm_weight.float() * self.query.float()).view(self.heads, hd)
        scores, values = [], []
        for s in sources:                                   # source-wise: no [S, B, T, C] fp32 tensor
            v = s.float()
            n = v * torch.rsqrt(v.square().mean(-1, keepdim=True) + self.eps)
            scores.append((n.unflatten(-1, (self.heads, hd)) * w).sum(-1))
            values.append(v.unflatten(-1, (self.heads, hd)))
        p = torch.softmax(torch.stack(scores, -1), -1)       # [..., heads, S]
        out = sum(p[..., i, None] * v for i, v in enumerate(values))
        return out.reshape(shape).to(sources[0].dtype)


class KimiBlock(nn.Module):
    def __init__(self, c: KimiConfig, layer_idx: int):
        super().__init__()
        self.is_kda = is_kda_layer(layer_idx, c.n_layer, c.kda_pattern, c.kda_force_final_global)
        self.attn = KimiDeltaAttention(c) if self.is_kda else GlobalGatedAttention(c)
        self.fc, self.proj = _lin(c.n_embd, 4 * c.n_embd), _lin(4 * c.n_embd, c.n_embd)

    def forward(self, x):
        x = x + self.attn(rms_norm(x))
        return x + self.proj(F.relu(self.fc(rms_norm(x))).square())


class KimiLM(nn.Module):
    def __init__(self, config: KimiConfig):
        super().__init__()
        c = self.config = config
        self.wte = nn.Embedding(c.vocab_size, c.n_embd)
        self.blocks = nn.ModuleList(KimiBlock(c, i) for i in range(c.n_layer))
        self.lm_head = _lin(c.n_embd, c.vocab_size)
        n_reads = (c.n_layer // c.attnres_block) if c.attnres_block else 0
        self.reads = nn.ModuleList(AttnResRead(c.n_embd, c.attnres_heads) for _ in range(n_reads))

    @torch.no_grad()
    def init_weights(self, std: float = 0.02):
        for n, p in self.named_parameters():
            if p.ndim >= 2:
                nn.init.normal_(p, std=std)
        for m in self.modules():
            if isinstance(m, nn.Linear) and m.bias is not None:
                m.bias.zero_()                       # a model built on the meta device has no defaults to fall back on
            if isinstance(m, KimiDeltaAttention):
                m.a_log.copy_(torch.empty_like(m.a_log).uniform_(1.0, 16.0).log())
                m.dt_bias.copy_(torch.empty_like(m.dt_bias).uniform_(-4.0, -1.0))
                m.output_norm_weight.fill_(1.0)
                for w in (m.q_conv, m.k_conv, m.v_conv):
                    nn.init.normal_(w, std=0.3)
            if isinstance(m, AttnResRead):
                m.query.zero_()
                m.norm_weight.fill_(1.0)

    def forward(self, ids, labels=None):
        c = self.config
        x = rms_norm(self.wte(ids))
        summaries = [x]
        for i, blk in enumerate(self.blocks):
            x = blk(x)
            if c.attnres_block and (i + 1) % c.attnres_block == 0:
                summaries.append(x)
                x = self.reads[(i + 1) // c.attnres_block - 1](*summaries)
        logits = self.lm_head(rms_norm(x)).float()
        logits = c.softcap * torch.tanh(logits / c.softcap)
        if labels is None:
            return logits
        return F.cross_entropy(logits.flatten(0, 1), labels.flatten(), ignore_index=-1)


from .protocol import attach_protocol  # noqa: E402  (after the classes it completes)

attach_protocol(KimiLM)
