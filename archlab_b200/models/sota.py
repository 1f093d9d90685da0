"""Component pool of published single-mechanism upgrades, their Pareto combinations, quantisation-aware
variants and the low-precision-friendly FOG family, all on one small decoder.

Mechanisms (choose any subset; the reference's pools are src/archlab/architectures/sota.py:48-385,
combinations.py:41-215 and fog.py:17-300):
  * ``dyt``         : Dynamic Tanh ``w * tanh(alpha x)`` instead of RMSNorm.
  * ``xielu``       : xIELU activation with trainable positive / negative curvature in the MLP.
  * ``canon``       : residual causal depthwise convolution (k = 4) before attention and MLP.
  * ``bov``         : bag-of-values - in the last ``bov_fraction`` of layers the value projection is replaced
                      by a token-indexed table initialised to W_V norm(embedding).
  * ``diff_attn``   : differential attention (two half-width softmax maps, learned lambda, sub-layer norm).
  * ``gated_relu`` / ``colu`` : parameter-matched gated feed-forward; CoLU rotates each cone of ``colu_dim`` channels.
  * ``qat``         : int8 per-token activations and int4 per-group weights as fake quantisation with a
                      straight-through estimator.
  * FOG: ``fog_variant`` in {opt, flash}: QK regularised by a frozen RMS norm or tanh, gain-initialised
    norms, and a ``QuantMonitor`` that records kurtosis / amax / non-finite fraction of tagged tensors.
"""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.attention import causal_attention
from .blocks import apply_rope, rms_norm, rope_tables

MECHANISMS = frozenset({"dyt", "xielu", "canon", "bov", "diff_attn", "gated_relu", "colu", "qat", "gated_attention",
                        "exclusive_attention"})


@dataclass(frozen=True)
class SotaConfig:
    vocab_size: int = 65536
    sequence_len: int = 2048
    n_layer: int = 14
    n_embd: int = 896
    n_head: int = 7
    mechanisms: tuple = ()
    bov_fraction: float = 0.25
    colu_dim: int = 4
    qat_group: int = 128
    fog_variant: str | None = None                    # None | "opt" | "flash"
    rope_theta: float = 100000.0

    def __post_init__(self):
        unknown = set(self.mechanisms) - MECHANISMS
        if unknown:
            raise ValueError(f"unknown mechanisms {sorted(unknown)}")
        if {"gated_relu", "colu"} <= set(self.mechanisms) or {"xielu", "colu"} <= set(self.mechanisms):
            raise ValueError("choose one feed-forward variant")
        if self.fog_variant not in (None, "opt", "flash"):
            raise ValueError("fog_variant must be opt or flash")
        if self.n_embd % self.n_head or (self.n_embd // self.n_head) % 4:
            raise ValueError("head width must be a multiple of 4")

    @property
    def head_dim(self):
        return self.n_embd // self.n_head

    def has(self, m):
        return m in self.mechanisms

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(vocab_size=128, sequence_len=64, n_layer=4, n_embd=64, n_head=4, qat_group=16), **kw})


# ------------------------------------------------------------------------------------------------
# building blocks
# ------------------------------------------------------------------------------------------------
class DynamicTanh(nn.Module):
    def __init__(self, width: int, alpha: float = 1.0):
        super().__init__()
        self.alpha, self.weight = nn.Parameter(torch.full((1,), alpha)), nn.Parameter(torch.ones(width))

    def forward(self, x):
        return self.weight.to(x.dtype) * torch.tanh(self.alpha.to(x.dtype) * x)


class XIELU(nn.Module):
    """x > 0: a_p x^2 + beta x;  x <= 0: a_n (expm1(min(x, -eps)) - x) + beta x, with a_p = softplus(.),
    a_n = beta + softplus(.)."""

    def __init__(self, alpha_p: float = 0.8, alpha_n: float = 0.8, beta: float = 0.5, eps: float = 1e-6):
        super().__init__()
        if alpha_n <= beta:
            raise ValueError("alpha_n must exceed beta")
        inv = lambda v: math.log(math.expm1(v))
        self.p, self.n = nn.Parameter(torch.tensor([inv(alpha_p)])), nn.Parameter(torch.tensor([inv(alpha_n - beta)]))
        self.beta, self.eps = beta, eps

    def forward(self, x):
        ap, an = F.softplus(self.p.float()).to(x.dtype), (self.beta + F.softplus(self.n.float())).to(x.dtype)
        neg = torch.minimum(x, x.new_tensor(-self.eps))
        return torch.where(x > 0, ap * x.square() + self.beta * x, an * torch.expm1(neg) - an * x + self.beta * x)


class CanonConv(nn.Module):
    def __init__(self, channels: int, k: int = 4):
        super().__init__()
        self.k = k
        self.weight = nn.Parameter(torch.empty(channels, 1, k))
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x):
        y = F.conv1d(F.pad(x.transpose(1, 2), (self.k - 1, 0)), self.weight.to(x.dtype), groups=x.size(-1))
        return x + y.transpose(1, 2)


def ste(original, quantized):
    return original + (quantized.to(original.dtype) - original).detach()


def fake_quant_int8_per_token(x):
    """Asymmetric dynamic int8 along the last dimension, straight-through gradient."""
    x32 = x.float()
    lo, hi = x32.amin(-1, keepdim=True), x32.amax(-1, keepdim=True)
    scale = ((hi - lo) / 255.0).clamp_min(torch.finfo(torch.float32).eps)
    zero = (-128.0 - lo / scale).round().clamp(-128, 127)
    q = ((x32 / scale).round() + zero).clamp(-128, 127)
    return ste(x, (q - zero) * scale)


def fake_quant_int4_per_group(w, group: int):
    """Symmetric signed int4 ([-8, 7], scale amax / 7) over groups of ``group`` input features."""
    if w.dim() != 2:
        raise ValueError("expected a matrix")
    o, i = w.shape
    pad = (-i) % group
    g = F.pad(w.float(), (0, pad)).view(o, -1, group)
    scale = (g.abs().amax(-1, keepdim=True) / 7.0).clamp_min(torch.finfo(torch.float32).eps)
    dq = ((g / scale).round().clamp(-8, 7) * scale).reshape(o, i + pad)[:, :i]
    return ste(w, dq)


class QATLinear(nn.Linear):
    def __init__(self, i, o, group: int = 128):
        super().__init__(i, o, bias=False)
        self.group = group

    def forward(self, x):
        return F.linear(fake_quant_int8_per_token(x), fake_quant_int4_per_group(self.weight, self.group).to(x.dtype))


def soft_colu(x, dim: int, eps: float = 1e-7):
    """Cone activation: channels form groups of ``dim`` = one axis t and dim-1 transverse w;
    t' = silu(t), w' = sigmoid(t' / (|w| + eps) - 1/2) w.  Axis channels come first."""
    if x.size(-1) % dim:
        raise ValueError("channels must divide the cone size")
    g = x.size(-1) // dim
    t, w = x.split([g, g * (dim - 1)], -1)
    w = w.unflatten(-1, (g, dim - 1))
    t_out = F.silu(t).unsqueeze(-1)
    radius = torch.linalg.vector_norm(w.float(), dim=-1, keepdim=True).to(w.dtype)
    return torch.cat([t_out.flatten(-2), (torch.sigmoid(t_out / (radius + eps) - 0.5) * w).flatten(-2)], -1)


def matched_gated_width(model_dim: int, multiple: int = 1) -> int:
    """Width of a three-matrix gated MLP with the parameters of the two-matrix 4x MLP (8d/3), rounded
    to ``multiple``."""
    w = round(8 * model_dim / 3)
    return max(multiple, round(w / multiple) * multiple)


def kurtosis(x):
    xf = x.float().reshape(-1)
    return xf.pow(4).mean() / xf.square().var(unbiased=False).clamp_min(1e-12)


class QuantMonitor:
    def __init__(self):
        self.enabled, self.records = False, defaultdict(list)

    def set_enabled(self, on: bool):
        self.enabled = on
        if not on:
            self.records.clear()

    def record(self, name: str, x):
        if not self.enabled:
            return
        xf = x.detach().float()
        self.records[f"{name}/kurtosis"].append(float(kurtosis(xf)))
        self.records[f"{name}/amax"].append(float(xf.abs().max()))
        self.records[f"{name}/nonfinite_frac"].append(float((~torch.isfinite(xf)).float().mean()))

    def consume(self) -> dict:
        out = {k: sum(v) / len(v) for k, v in self.records.items() if v}
        self.records.clear()
        return out


# ------------------------------------------------------------------------------------------------
# model
# ------------------------------------------------------------------------------------------------
class PoolAttention(nn.Module):
    def __init__(self, c: SotaConfig, layer: int):
        super().__init__()
        self.c, self.layer = c, layer
        lin = (lambda i, o: QATLinear(i, o, c.qat_group)) if c.has("qat") else (lambda i, o: nn.Linear(i, o, bias=False))
        self.q, self.k, self.o = lin(c.n_embd, c.n_embd), lin(c.n_embd, c.n_embd), lin(c.n_embd, c.n_embd)
        start = c.n_layer - max(1, int(c.n_layer * c.bov_fraction))
        self.bov = c.has("bov") and layer >= start
        if self.bov:
            self.value_table = nn.Embedding(c.vocab_size, c.n_embd)
        else:
            self.v = lin(c.n_embd, c.n_embd)
        if c.has("gated_attention"):
            # query-dependent head-wise sigmoid gate on the attention output (src/archlab/architectures/sota.py:162-163, 299-301)
            self.output_gate = nn.Linear(c.n_embd, c.n_head, bias=False)
        if c.has("diff_attn"):
            half = c.head_dim // 2
            self.lambda_init = 0.8 - 0.6 * math.exp(-0.3 * layer)
            self.lq1, self.lk1, self.lq2, self.lk2 = (nn.Parameter(torch.randn(half) * 0.1) for _ in range(4))
            self.subln = nn.Parameter(torch.ones(c.head_dim))

    @torch.no_grad()
    def init_bov(self, embedding: nn.Embedding, v_proj: nn.Linear) -> None:
        """value_table[token] = W_V norm(embedding[token]): at initialisation the table reproduces the projection."""
        for s in range(0, embedding.weight.size(0), 2048):
            self.value_table.weight[s:s + 2048].copy_(v_proj(rms_norm(embedding.weight[s:s + 2048])))

    def forward(self, x, ids, cos, sin, monitor=None):
        c = self.c
        B, T, _ = x.shape
        H, D = c.n_head, c.head_dim
        q, k = self.q(x).view(B, T, H, D), self.k(x).view(B, T, H, D)
        v = (self.value_table(ids) if self.bov else self.v(x)).view(B, T, H, D).to(x.dtype)
        if c.has("diff_attn"):
            half = D // 2
            cs, sn = cos[:, : half // 2], sin[:, : half // 2]
            parts = []
            for t in (q, k):
                t = t.view(B, T, H, 2, half)
                parts += [rms_norm(apply_rope(t[..., 0, :], cs, sn)) * 1.2, rms_norm(apply_rope(t[..., 1, :], cs, sn)) * 1.2]
            q1, q2, k1, k2 = parts
            att = lambda a, b: F.scaled_dot_product_attention(a.transpose(1, 2), b.transpose(1, 2), v.transpose(1, 2),
                                                              is_causal=True).transpose(1, 2)
            lam = (torch.exp((self.lq1 * self.lk1).sum().float()) - torch.exp((self.lq2 * self.lk2).sum().float())
                   + self.lambda_init).to(x.dtype)
            y = rms_norm(att(q1, k1) - lam * att(q2, k2)) * self.subln.to(x.dtype) * (1.0 - self.lambda_init)
        else:
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            if c.fog_variant == "flash":
                q, k = torch.tanh(q), torch.tanh(k)
            elif c.fog_variant == "opt":
                q, k = rms_norm(q), rms_norm(k)
            else:
                q, k = rms_norm(q) * 1.2, rms_norm(k) * 1.2
            if monitor is not None:
                monitor.record(f"layer{self.layer}/q", q)
                monitor.record(f"layer{self.layer}/k", k)
            y = causal_attention(q, k, v)
            if c.has("gated_attention"):
                y = y * torch.sigmoid(self.output_gate(x)).unsqueeze(-1).to(y.dtype)
            elif c.has("exclusive_attention"):
                # the output keeps only what is orthogonal to the token's own value (sota.py:302-304)
                vd = F.normalize(v, dim=-1)
                y = y - (y * vd).sum(-1, keepdim=True) * vd
        return self.o(y.reshape(B, T, -1))


class PoolMLP(nn.Module):
    def __init__(self, c: SotaConfig):
        super().__init__()
        self.c = c
        lin = (lambda i, o: QATLinear(i, o, c.qat_group)) if c.has("qat") else (lambda i, o: nn.Linear(i, o, bias=False))
        self.gated = c.has("gated_relu") or c.has("colu")
        width = matched_gated_width(c.n_embd, c.colu_dim if c.has("colu") else 1) if self.gated else 4 * c.n_embd
        self.fc, self.proj = lin(c.n_embd, width), lin(width, c.n_embd)
        if self.gated:
            self.up = lin(c.n_embd, width)
        self.act = XIELU() if c.has("xielu") else None
        self.last_active_fraction = None

    def forward(self, x):
        h = self.fc(x)
        if self.c.has("colu"):
            h = soft_colu(h, self.c.colu_dim) * self.up(x)
        elif self.gated:
            a = F.relu(h)
            self.last_active_fraction = float((a > 0).float().mean())
            h = a * self.up(x)
        elif self.act is not None:
            h = self.act(h)
        else:
            h = F.relu(h).square()
        return self.proj(h)


class PoolBlock(nn.Module):
    def __init__(self, c: SotaConfig, layer: int):
        super().__init__()
        self.c = c
        if c.has("dyt"):
            self.n1, self.n2 = DynamicTanh(c.n_embd), DynamicTanh(c.n_embd)
        elif c.fog_variant is not None:                      # gain-initialised norms keep early activations small
            gain = 1.0 / math.sqrt(2 * (layer + 1))
            self.g1, self.g2 = nn.Parameter(torch.full((c.n_embd,), gain)), nn.Parameter(torch.full((c.n_embd,), gain))
        self.attn, self.mlp = PoolAttention(c, layer), PoolMLP(c)
        if c.has("canon"):
            self.canon_a, self.canon_m = CanonConv(c.n_embd), CanonConv(c.n_embd)

    def _norm(self, x, which):
        if self.c.has("dyt"):
            return (self.n1 if which == 1 else self.n2)(x)
        if self.c.fog_variant is not None:
            return rms_norm(x, self.g1 if which == 1 else self.g2)
        return rms_norm(x)

    def forward(self, x, ids, cos, sin, monitor=None):
        h = self._norm(x, 1)
        if self.c.has("canon"):
            h = self.canon_a(h)
        x = x + self.attn(h, ids, cos, sin, monitor)
        h = self._norm(x, 2)
        if self.c.has("canon"):
            h = self.canon_m(h)
        if monitor is not None:
            monitor.record(f"layer{self.attn.layer}/mlp_in", h)
        return x + self.mlp(h)


class SotaLM(nn.Module):
    def __init__(self, config: SotaConfig):
        super().__init__()
        c = self.config = config
        self.embed = nn.Embedding(c.vocab_size, c.n_embd)
        self.layers = nn.ModuleList(PoolBlock(c, i) for i in range(c.n_layer))
        self.lm_head = nn.Linear(c.n_embd, c.vocab_size, bias=False)
        self.monitor = QuantMonitor()

    def init_weights(self, std: float = 0.02):
        for n, p in self.named_parameters():
            if p.dim() == 2 and "value_table" not in n:
                nn.init.normal_(p, std=std)
        if self.config.has("bov"):
            for blk in self.layers:
                if blk.attn.bov:
                    tmp = nn.Linear(self.config.n_embd, self.config.n_embd, bias=False)
                    nn.init.normal_(tmp.weight, std=std)
                    blk.attn.init_bov(self.embed, tmp)

    def architecture_state(self) -> dict:
        c = self.config
        return {"mechanisms": sorted(c.mechanisms), "fog_variant": c.fog_variant,
                "bov_layers": [i for i, b in enumerate(self.layers) if b.attn.bov],
                "parameters": sum(p.numel() for p in self.parameters())}

    def forward(self, ids, labels=None):
        c = self.config
        cos, sin = rope_tables(ids.size(1), c.head_dim, c.rope_theta, ids.device)
        x = rms_norm(self.embed(ids))
        mon = self.monitor if self.monitor.enabled else None
        for blk in self.layers:
            x = blk(x, ids, cos, sin, mon)
        logits = 15.0 * torch.tanh(self.lm_head(rms_norm(x)).float() / 15.0)
        if labels is None:
            return logits
        return F.cross_entropy(logits.flatten(0, 1), labels.flatten(), ignore_index=-1)


PARETO_COMBOS = {
    "canon_xielu": ("canon", "xielu"),
    "canon_diff": ("canon", "diff_attn"),
    "canon_bov_gated": ("canon", "bov", "gated_relu"),
    "qat_canon_gated": ("qat", "canon", "gated_relu"),
    "dyt_colu": ("dyt", "colu"),
}


def combo_config(name: str, **kw) -> SotaConfig:
    if name not in PARETO_COMBOS:
        raise ValueError(f"unknown combination {name!r}")
    return SotaConfig(mechanisms=PARETO_COMBOS[name], **kw)


from .protocol import attach_protocol  # noqa: E402  (after the classes it completes)

attach_protocol(SotaLM)
