"""Additive mechanism adapters on multi-stream residual states, and the triadic switch.

``StreamAdapter`` is one zero-initialised branch on a packed n-stream state ``[B, T, n * C]``: gated-residual
read of the streams (group norm, low-rank sigmoid mix) -> mechanism -> sigmoid output gate -> zero-init output
projection -> injection into every stream with 2*sigmoid weights.  At installation the model's function is
unchanged.  Mechanisms: ``simplicial`` (q / k1 / k2 with zero-centred RMSNorm and partial RoPE, v1 / v2,
windowed 2-simplicial core), ``normal`` (parameter-matched windowed softmax attention), ``linsimp`` (positive
random-feature linear attention), ``triadic`` (joint-key gated delta rule over E feature slices) and ``mixer``
(parameter-matched gated MLP, the no-attention control).  These are the arms of the reference's Flash-Next
and V4.1 adapter studies (src/archlab/architectures/simplicial_adapter.py:88-156,
deepseek_v41_adapters.py) behind one class.

``TriadicSwitch`` replaces a gated-delta-rule mixer by its triadic form and inherits the teacher's q / k / v /
gate / output weights; the second key and query are new (zero weights, bias such that they start as the
constant 1 / sqrt(E)), so the switched layer starts as the teacher
(src/archlab/architectures/qwen35_switch.py:150-218).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import delta_rule, linsimp, local_attention, triadic
from ..ops import simplicial as sx
from .blocks import GatedStreamResidual, GroupRMSNorm, apply_rope, rope_tables

MECHANISMS = ("simplicial", "normal", "linsimp", "triadic", "mixer")


@dataclass(frozen=True)
class AdapterConfig:
    hidden_size: int
    streams: int = 4
    mechanism: str = "simplicial"
    heads: int = 4
    kv_heads: int = 1
    head_dim: int = 128
    short_window: int = 16
    long_window: int = 512
    rotary_fraction: float = 0.25
    rope_theta: float = 1e6
    low_rank: int = 64
    feature_rank: int = 128
    triadic_slices: int = 4
    rms_eps: float = 1e-6

    def __post_init__(self):
        if self.mechanism not in MECHANISMS:
            raise ValueError(f"unknown adapter mechanism {self.mechanism!r}")
        if self.heads % self.kv_heads:
            raise ValueError("query heads must be a multiple of KV heads")


def _lin(i, o):
    return nn.Linear(i, o, bias=False)


class StreamAdapter(nn.Module):
    def __init__(self, c: AdapterConfig, *, seed: int = 0):
        super().__init__()
        self.c = c
        W, q, kv = c.hidden_size, c.heads * c.head_dim, c.kv_heads * c.head_dim
        with torch.random.fork_rng(devices=[]):
            torch.manual_seed(seed)
            self.read = GatedStreamResidual(W, c.streams, c.low_rank, c.rms_eps, zero_centered=True)
            m = c.mechanism
            if m == "mixer":
                # same parameter count as the simplicial arm: q + gate + 4 kv + out  ->  three matrices of width `inter`
                inter = max(8, round((3 * W * q + 4 * W * kv) / (3 * W) / 8) * 8)
                self.gate_proj, self.up_proj, self.output = _lin(W, inter), _lin(W, inter), _lin(inter, W)
            else:
                self.q, self.output_gate, self.output = _lin(W, q), _lin(W, q), _lin(q, W)
                n_kv = {"simplicial": 2, "linsimp": 2, "triadic": 1, "normal": 1}[m]
                self.keys = nn.ModuleList(_lin(W, kv) for _ in range(n_kv))
                self.values = nn.ModuleList(_lin(W, kv) for _ in range(n_kv))
                self.q_norm = GroupRMSNorm(c.head_dim, 1, c.rms_eps, zero_centered=True)
                self.k_norms = nn.ModuleList(GroupRMSNorm(c.head_dim, 1, c.rms_eps, zero_centered=True) for _ in range(n_kv))
                if m == "normal":                              # spend the second K/V stream's parameters on width instead
                    self.extra = _lin(W, 2 * kv)
                if m == "linsimp":
                    self.register_buffer("omega", linsimp.orthogonal_feature_bank(c.heads, c.head_dim, c.feature_rank, seed=seed))
                if m == "triadic":
                    E = c.triadic_slices
                    self.k2, self.q2 = nn.Linear(W, c.heads * E), nn.Linear(W, c.heads * E)
                    self.decay, self.beta = _lin(W, c.heads), _lin(W, c.heads)
            for mod in self.modules():
                if isinstance(mod, nn.Linear):
                    nn.init.normal_(mod.weight, std=0.02)
                    if mod.bias is not None:
                        nn.init.zeros_(mod.bias)
            nn.init.zeros_(self.output.weight)

    def project(self, x: torch.Tensor, offset: int = 0):
        """Normalised, rotated queries and keys and the values of ``x`` [B, T, W] whose first token sits at absolute
        position ``offset`` (the incremental serving form projects one chunk at a time).  The ``normal`` arm folds its
        widening projections into its single key / value stream here."""
        c = self.c
        B, T, _ = x.shape
        rot = int(c.head_dim * c.rotary_fraction) // 2 * 2
        cos, sin = rope_tables(T, max(rot, 2), c.rope_theta, x.device, offset=offset)
        rope = (lambda t: apply_rope(t, cos, sin, rot_dim=rot)) if rot else (lambda t: t)
        q = rope(self.q_norm(self.q(x).view(B, T, c.heads, c.head_dim)))
        ks = [rope(n(k(x).view(B, T, c.kv_heads, c.head_dim))) for k, n in zip(self.keys, self.k_norms)]
        vs = [v(x).view(B, T, c.kv_heads, c.head_dim) for v in self.values]
        if c.mechanism == "normal":
            ek, ev = self.extra(x).view(B, T, 2, c.kv_heads, c.head_dim).unbind(2)     # the matched parameters widen K and V
            ks, vs = [ks[0] + rope(self.k_norms[0](ek))], [vs[0] + ev]
        return q, ks, vs

    def attend(self, q, ks, vs):
        """Windowed core of the ``simplicial`` and ``normal`` arms; keys may be longer than queries (cached prefix
        first): the queries are the LAST ``q.shape[1]`` positions of the key sequence."""
        c, T, S = self.c, q.shape[1], ks[0].shape[1]
        if S != T:                                                             # left-pad queries; their rows are dropped below
            q = torch.cat([q.new_zeros(q.shape[0], S - T, *q.shape[2:]), q], dim=1)
        if c.mechanism == "simplicial":
            w2 = min(S, c.long_window)
            y = sx.simplicial_attention(q, ks[0], ks[1], vs[0], vs[1], min(c.short_window, w2), w2)
        else:
            y = local_attention.local_attention(q, ks[0], vs[0], min(S, c.long_window))
        return y[:, S - T:]

    def finish(self, x, y):
        return self.output(y.reshape(x.shape[0], x.shape[1], -1).to(x.dtype) * torch.sigmoid(self.output_gate(x)))

    def branch(self, x: torch.Tensor) -> torch.Tensor:
        c, m = self.c, self.c.mechanism
        B, T, _ = x.shape
        if m == "mixer":
            return self.output(F.silu(self.gate_proj(x)) * self.up_proj(x))
        q, ks, vs = self.project(x)
        if m in ("simplicial", "normal"):
            y = self.attend(q, ks, vs)
        elif m == "linsimp":
            y = linsimp.linsimp_attention(q, ks[0], ks[1], vs[0], vs[1], self.omega, window=min(T, c.short_window))
        else:
            E, rep = c.triadic_slices, c.heads // c.kv_heads
            k, v = ks[0].repeat_interleave(rep, 2), vs[0].repeat_interleave(rep, 2)
            k2 = F.normalize(self.k2(x).view(B, T, c.heads, E).float(), dim=-1)
            q2 = F.normalize(self.q2(x).view(B, T, c.heads, E).float(), dim=-1)
            g = -F.softplus(self.decay(x).float()).unsqueeze(-1).expand(B, T, c.heads, E)      # one decay per head, shared by its slices
            y = triadic.triadic_gdn_attention(F.normalize(q.float(), dim=-1), F.normalize(k.float(), dim=-1), v.float(), k2, q2, g,
                                              torch.sigmoid(self.beta(x).float())).to(x.dtype)
        return self.finish(x, y)

    def forward(self, packed: torch.Tensor) -> torch.Tensor:
        x, packed, w = self.read(packed)
        return GatedStreamResidual.inject(packed, self.branch(x.to(packed.dtype)), w.to(packed.dtype))


def parameter_report(c: AdapterConfig) -> dict:
    """Parameter counts of every arm at the same geometry (the controls must match the simplicial arm closely)."""
    out = {}
    for m in MECHANISMS:
        a = StreamAdapter(AdapterConfig(**{**c.__dict__, "mechanism": m}))
        out[m] = sum(p.numel() for p in a.parameters())
    return out


class TriadicSwitch(nn.Module):
    """Gated delta rule -> triadic gated delta rule over ``E`` feature slices, starting as the teacher."""

    def __init__(self, hidden: int, heads: int, key_dim: int, value_dim: int, slices: int = 4):
        super().__init__()
        self.h, self.kd, self.vd, self.E = heads, key_dim, value_dim, slices
        self.q, self.k, self.v = _lin(hidden, heads * key_dim), _lin(hidden, heads * key_dim), _lin(hidden, heads * value_dim)
        self.ba = _lin(hidden, 2 * heads)
        self.a_log = nn.Parameter(torch.zeros(heads))
        self.dt_bias = nn.Parameter(torch.zeros(heads))
        self.o = _lin(heads * value_dim, hidden)
        self.k2, self.q2 = nn.Linear(hidden, heads * slices), nn.Linear(hidden, heads * slices)
        with torch.no_grad():
            for m in (self.k2, self.q2):
                m.weight.zero_()
                m.bias.fill_(1.0)                              # normalised below: every slice starts at 1 / sqrt(E)

    @torch.no_grad()
    def inherit(self, teacher) -> None:
        """``teacher`` exposes q / k / v / ba / o linears and a_log / dt_bias of matching shapes."""
        for name in ("q", "k", "v", "ba", "o"):
            getattr(self, name).weight.copy_(getattr(teacher, name).weight)
        self.a_log.copy_(teacher.a_log)
        self.dt_bias.copy_(teacher.dt_bias)

    def forward(self, x):
        B, T, _ = x.shape
        q = F.normalize(self.q(x).view(B, T, self.h, self.kd).float(), dim=-1)
        k = F.normalize(self.k(x).view(B, T, self.h, self.kd).float(), dim=-1)
        v = self.v(x).view(B, T, self.h, self.vd).float()
        b_logit, d_logit = self.ba(x).float().chunk(2, -1)
        g = -self.a_log.float().exp() * F.softplus(d_logit + self.dt_bias.float())
        k2 = F.normalize(self.k2(x).view(B, T, self.h, self.E).float(), dim=-1)
        q2 = F.normalize(self.q2(x).view(B, T, self.h, self.E).float(), dim=-1)
        # with k2 = q2 = const unit vector the E slices hold identical copies scaled by 1/E each way: the read
        # sums E * (1/sqrt(E))^2 ... = the plain delta rule
        y = triadic.triadic_gdn_attention(q, k, v, k2, q2, g.unsqueeze(-1).expand(B, T, self.h, self.E), torch.sigmoid(b_logit),
                                          scale=self.kd ** -0.5)
        return self.o(y.reshape(B, T, -1).to(x.dtype))


class PlainDeltaMixer(nn.Module):
    """The teacher form the switch starts from (same parameter names)."""

    def __init__(self, hidden: int, heads: int, key_dim: int, value_dim: int):
        super().__init__()
        self.h, self.kd, self.vd = heads, key_dim, value_dim
        self.q, self.k, self.v = _lin(hidden, heads * key_dim), _lin(hidden, heads * key_dim), _lin(hidden, heads * value_dim)
        self.ba = _lin(hidden, 2 * heads)
        self.a_log = nn.Parameter(torch.zeros(heads))
        self.dt_bias = nn.Parameter(torch.zeros(heads))
        self.o = _lin(heads * value_dim, hidden)

    def forward(self, x):
        B, T, _ = x.shape
        b_logit, d_logit = self.ba(x).float().chunk(2, -1)
        g = -self.a_log.float().exp() * F.softplus(d_logit + self.dt_bias.float())
        y = delta_rule.gated_delta_reference(self.q(x).view(B, T, self.h, self.kd), self.k(x).view(B, T, self.h, self.kd),
                                             self.v(x).view(B, T, self.h, self.vd), g, torch.sigmoid(b_logit))
        return self.o(y.reshape(B, T, -1).to(x.dtype))
