"""Frontier mechanism pool: one controlled backbone, many swappable token mixers / feed-forwards.

Each variant changes exactly one mechanism of a small pre-norm decoder (QK-normed rotary attention +
ReLU^2 MLP): relative-position attention with a learned distance bank, short causal convolutions on
K/V or on the residual stream, a 5:1 sliding/full hybrid, partial (25 %) RoPE, zero-centred RMSNorm,
the sigmoid-tanh GLU, shared multi-token prediction, attention sinks, gated delta rule mixers,
compressed-sequence attention (light: 4-token blocks with an overlapping second stream; heavy:
128-token blocks), multi-latent attention, grouped differential latent attention and annealed
hyper-connections.  The list and the parameterisations follow the reference's frontier pool
(src/archlab/architectures/frontier.py:30-52 variants, :160-182 short convolution, :360-484 compressed
attention, :486-529 MLA, :531-598 GDLA, :600-619 SiTU-GLU, :637-803 attention variants, :845-879 MTP);
here every mixer is a small strategy class with the signature ``mixer(x, cos, sin) -> y``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import delta_rule
from ..ops.attention import causal_attention
from .blocks import RMSNorm, apply_rope, rms_norm, rope_tables

VARIANTS = ("baseline", "inkling_relative_attention", "inkling_sconv_kv", "inkling_sconv_residual", "hybrid_swa_5_1_w512",
            "partial_rope_25", "zero_centered_rmsnorm", "kimi_situ_glu", "shared_mtp3", "attention_sink", "qwen_gdn",
            "deepseek_csa", "deepseek_hca", "glm_mla", "motif_gdla", "motif_mhc")


@dataclass(frozen=True)
class FrontierConfig:
    vocab_size: int = 65536
    sequence_len: int = 2048
    n_layer: int = 14
    n_embd: int = 896
    n_head: int = 7
    variant: str = "baseline"
    relative_dim: int = 16
    relative_extent: int = 1024
    sconv_kernel: int = 4
    mtp_depth: int = 3
    mtp_weight: float = 0.1
    hc_streams: int = 4
    hc_sinkhorn_iters: int = 20
    hc_anneal_steps: int = 1907
    rope_theta: float = 100000.0

    def __post_init__(self):
        if self.variant not in VARIANTS:
            raise ValueError(f"unknown frontier variant {self.variant!r}")
        if self.n_embd % self.n_head:
            raise ValueError("width must divide into heads")
        if self.variant == "partial_rope_25" and ((self.n_embd // self.n_head) // 4) % 2:
            raise ValueError("25% partial RoPE needs an even rotary width")

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @classmethod
    def tiny(cls, **kw):
        return cls(**{**dict(vocab_size=128, sequence_len=64, n_layer=2, n_embd=64, n_head=4, relative_extent=32), **kw})


def _lin(i, o):
    return nn.Linear(i, o, bias=False)


def _masked_attention(q, k, v, allowed, sink=None):
    """q [B,T,H,D], k/v [B,S,H,D], allowed [T,S] bool, optional per-head sink logit (a key of value 0)."""
    s = torch.einsum("bthd,bshd->bhts", q.float(), k.float()) * q.size(-1) ** -0.5
    s = s.masked_fill(~allowed.view(1, 1, *allowed.shape), float("-inf"))
    if sink is not None:
        s = torch.cat([s, sink.float().view(1, -1, 1, 1).expand(s.size(0), -1, s.size(2), 1)], -1)
    p = s.softmax(-1)
    if sink is not None:
        p = p[..., :-1]
    return torch.einsum("bhts,bshd->bthd", p, v.float()).to(v.dtype)


class ShortConv(nn.Module):
    """fp32 residual causal depthwise convolution; the weight is a [C, k] matrix (Muon treats it as one)."""

    def __init__(self, channels: int, k: int = 4):
        super().__init__()
        self.k = k
        self.weight = nn.Parameter(torch.empty(channels, k))
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x):
        r = x.float()
        y = F.conv1d(F.pad(r.transpose(1, 2), (self.k - 1, 0)), self.weight.float().unsqueeze(1), groups=r.size(-1))
        return (r + y.transpose(1, 2)).to(x.dtype)


class StandardAttention(nn.Module):
    """Baseline mixer and its one-line variants (window, rotary fraction, sink, K/V convolution, relative bank)."""

    def __init__(self, c: FrontierConfig, layer: int):
        super().__init__()
        self.c, self.layer = c, layer
        self.q, self.k, self.v, self.o = (_lin(c.n_embd, c.n_embd) for _ in range(4))
        v = c.variant
        self.rot = c.head_dim // 4 if v == "partial_rope_25" else c.head_dim
        self.window = 512 if (v == "hybrid_swa_5_1_w512" and (layer + 1) % 6 != 0) else -1
        if v == "inkling_sconv_kv":
            self.k_conv, self.v_conv = ShortConv(c.n_embd, c.sconv_kernel), ShortConv(c.n_embd, c.sconv_kernel)
        if v == "inkling_relative_attention":
            self.r_proj = _lin(c.n_embd, c.n_head * c.relative_dim)
            self.bank = nn.Parameter(torch.randn(c.relative_dim, c.relative_extent) * 0.02)
        if v == "attention_sink":
            self.sink = nn.Parameter(torch.zeros(c.n_head))

    def forward(self, x, cos, sin):
        c, v = self.c, self.c.variant
        B, T, _ = x.shape
        kf, vf = self.k(x), self.v(x)
        if v == "inkling_sconv_kv":
            kf, vf = self.k_conv(kf), self.v_conv(vf)
        q, k, val = (t.view(B, T, c.n_head, c.head_dim) for t in (self.q(x), kf, vf))
        q = rms_norm(apply_rope(q, cos[:, : self.rot // 2], sin[:, : self.rot // 2], rot_dim=self.rot)) * 1.2
        k = rms_norm(apply_rope(k, cos[:, : self.rot // 2], sin[:, : self.rot // 2], rot_dim=self.rot)) * 1.2
        pos = torch.arange(T, device=x.device)
        dist = pos[:, None] - pos[None, :]
        if v == "inkling_relative_attention":
            s = torch.einsum("bthd,bshd->bhts", q.float(), k.float()) * c.head_dim ** -0.5
            rel = self.r_proj(x).view(B, T, c.n_head, c.relative_dim).float()
            logits = torch.einsum("bthr,re->bhte", rel, self.bank.float())            # per query: bias for each distance
            idx = dist.clamp(0, c.relative_extent - 1).view(1, 1, T, T).expand(B, c.n_head, -1, -1)
            bias = logits.gather(-1, idx).masked_fill(~((dist >= 0) & (dist < c.relative_extent)).view(1, 1, T, T), 0.0)
            p = (s + bias).masked_fill(~(dist >= 0).view(1, 1, T, T), float("-inf")).softmax(-1)
            y = torch.einsum("bhts,bshd->bthd", p, val.float()).to(x.dtype)
        elif v == "attention_sink":
            y = _masked_attention(q, k, val, dist >= 0, self.sink)
        else:
            y = causal_attention(q, k, val, self.window)
        return self.o(y.reshape(B, T, -1))


class GatedDeltaMixer(nn.Module):
    """Short convolution -> gated delta rule (scalar decay) -> per-head norm -> output gate."""

    def __init__(self, c: FrontierConfig, layer: int):
        super().__init__()
        self.c = c
        self.qkv = _lin(c.n_embd, 3 * c.n_embd)
        self.conv = nn.Parameter(torch.randn(3 * c.n_embd, c.sconv_kernel) * 0.1)
        self.ba = _lin(c.n_embd, 2 * c.n_head)
        self.a_log = nn.Parameter(torch.zeros(c.n_head))
        self.dt_bias = nn.Parameter(torch.full((c.n_head,), -4.0))
        self.z, self.o = _lin(c.n_embd, c.n_embd), _lin(c.n_embd, c.n_embd)
        self.norm = RMSNorm(c.head_dim)

    def forward(self, x, cos, sin):
        c = self.c
        B, T, _ = x.shape
        q, k, v = (t.view(B, T, c.n_head, c.head_dim) for t in delta_rule.causal_conv1d(self.qkv(x), self.conv).chunk(3, -1))
        b_logit, d_logit = self.ba(x).chunk(2, -1)
        decay = -self.a_log.float().exp() * F.softplus(d_logit.float() + self.dt_bias.float())
        y = delta_rule.gated_delta_rule(q, k, v, decay, b_logit.sigmoid()).to(x.dtype)
        return self.o((self.norm(y) * F.silu(self.z(x).view_as(y))).flatten(-2))


class CompressedAttention(nn.Module):
    """One shared K = V stream: learned softmax pooling of ``m``-token blocks (light: m = 4 with a second,
    one-block-delayed stream; heavy: m = 128) next to a 128-token local window; rotary on the trailing
    channels, removed again from the output (the keys are the values)."""

    def __init__(self, c: FrontierConfig, layer: int, heavy: bool):
        super().__init__()
        self.c, self.heavy = c, heavy
        self.m, self.local = (128 if heavy else 4), 128
        D = c.head_dim
        self.rot = 64 if D == 128 else max(2, D // 2) // 2 * 2
        self.q_down, self.q_up = _lin(c.n_embd, c.n_embd // 2), _lin(c.n_embd // 2, c.n_embd)
        self.c_a, self.z_a = _lin(c.n_embd, D), _lin(c.n_embd, D)
        self.bias_a = nn.Parameter(torch.zeros(self.m, D))
        if not heavy:
            self.c_b, self.z_b = _lin(c.n_embd, D), _lin(c.n_embd, D)
            self.bias_b = nn.Parameter(torch.zeros(self.m, D))
        self.head_out = nn.Parameter(torch.randn(c.n_head, D, D) * D ** -0.5)
        self.o = _lin(c.n_embd, c.n_embd)

    def _blocks(self, t, fill=0.0):
        pad = (-t.size(1)) % self.m
        if pad:
            t = F.pad(t, (0, 0, 0, pad), value=fill)
        return t.unflatten(1, (-1, self.m))

    def _compress(self, x):
        ca, za = self._blocks(self.c_a(x)), self._blocks(self.z_a(x), float("-inf")).float() + self.bias_a.float()
        if self.heavy:
            return (za.softmax(2).to(ca.dtype) * ca).sum(2)
        cb, zb = self._blocks(self.c_b(x)), self._blocks(self.z_b(x), float("-inf")).float()
        cb = torch.cat([torch.zeros_like(cb[:, :1]), cb[:, :-1]], 1)                       # previous block's second stream
        zb = torch.cat([torch.full_like(zb[:, :1], float("-inf")), zb[:, :-1]], 1) + self.bias_b.float()
        w = torch.cat([za, zb], 2).softmax(2).to(ca.dtype)
        return (w[:, :, : self.m] * ca).sum(2) + (w[:, :, self.m:] * cb).sum(2)

    def _rope_tail(self, t, cos, sin, inverse=False):
        r = self.rot
        tail = apply_rope(t[..., -r:], cos[:, : r // 2], (-sin if inverse else sin)[:, : r // 2])
        return torch.cat([t[..., :-r], tail], -1)

    def forward(self, x, cos, sin):
        c = self.c
        B, T, _ = x.shape
        q = self._rope_tail(rms_norm(self.q_up(self.q_down(x)).view(B, T, c.n_head, c.head_dim)), cos, sin)
        comp = rms_norm(self._compress(x))
        G = comp.size(1)
        bpos = (torch.arange(G, device=x.device) * self.m + self.m - 1).clamp_max(T - 1)
        comp = self._rope_tail(comp.unsqueeze(2), cos[bpos], sin[bpos]).squeeze(2)
        local = self._rope_tail(rms_norm(self.c_a(x)).unsqueeze(2), cos, sin).squeeze(2)
        kv = torch.cat([comp, local], 1).unsqueeze(2).expand(-1, -1, c.n_head, -1)
        tpos = torch.arange(T, device=x.device)
        comp_ok = torch.arange(G, device=x.device)[None, :] < (tpos // self.m)[:, None]      # only fully past blocks
        d = tpos[:, None] - tpos[None, :]
        y = _masked_attention(q, kv, kv, torch.cat([comp_ok, (d >= 0) & (d < self.local)], 1))
        y = self._rope_tail(y, cos, sin, inverse=True)
        y = torch.einsum("bthd,hde->bthe", y, self.head_out.to(y.dtype))
        return self.o(y.reshape(B, T, -1))


class MultiLatentAttention(nn.Module):
    def __init__(self, c: FrontierConfig, layer: int):
        super().__init__()
        self.c = c
        L = min(256, c.n_embd)
        self.q_down, self.kv_down = _lin(c.n_embd, L), _lin(c.n_embd, L)
        self.q_up, self.k_up, self.v_up = (_lin(L, c.n_embd) for _ in range(3))
        self.o = _lin(c.n_embd, c.n_embd)

    def forward(self, x, cos, sin):
        c = self.c
        B, T, _ = x.shape
        ql, kvl = self.q_down(x), self.kv_down(x)
        q, k, v = (p(t).view(B, T, c.n_head, c.head_dim) for p, t in ((self.q_up, ql), (self.k_up, kvl), (self.v_up, kvl)))
        q, k = rms_norm(apply_rope(q, cos, sin)) * 1.2, rms_norm(apply_rope(k, cos, sin)) * 1.2
        return self.o(causal_attention(q, k, v).reshape(B, T, -1))


class GroupedDifferentialLatentAttention(nn.Module):
    """n_head - 1 signal heads and one noise head over a single latent key/value head:
    out = gate * (signal - sigmoid(lambda) * noise)."""

    def __init__(self, c: FrontierConfig, layer: int):
        super().__init__()
        self.c = c
        D = c.head_dim
        self.sig, self.rot = c.n_head - 1, D // 2
        self.content, self.L = D - self.rot, min(256, c.n_embd)
        self.q_down, self.q_up = _lin(c.n_embd, self.L), _lin(self.L, c.n_head * D)
        self.kv_down, self.kv_up = _lin(c.n_embd, self.L + self.rot), _lin(self.L, self.content + D)
        self.lam, self.gate = _lin(c.n_embd, self.sig), _lin(self.L, self.sig * D)
        self.o = _lin(self.sig * D, c.n_embd)

    def forward(self, x, cos, sin):
        c, D = self.c, self.c.head_dim
        B, T, _ = x.shape
        ql = rms_norm(self.q_down(x))
        q = self.q_up(ql).view(B, T, c.n_head, D)
        kvl, rk = self.kv_down(x).split([self.L, self.rot], -1)
        ck, v = self.kv_up(rms_norm(kvl)).split([self.content, D], -1)
        cs, sn = cos[:, : self.rot // 2], sin[:, : self.rot // 2]
        q = torch.cat([q[..., : self.content], apply_rope(q[..., self.content:], cs, sn)], -1)
        k = torch.cat([ck.view(B, T, 1, self.content), apply_rope(rk.view(B, T, 1, self.rot), cs, sn)], -1)
        q, k, v = rms_norm(q) * 1.2, rms_norm(k) * 1.2, v.view(B, T, 1, D)
        both = causal_attention(q, k, v)                                # grouped-query: one shared K/V head
        signal, noise = both[:, :, : self.sig], both[:, :, self.sig:]
        diff = signal - torch.sigmoid(self.lam(x)).unsqueeze(-1) * noise
        return self.o((torch.sigmoid(self.gate(ql)).view_as(diff) * diff).reshape(B, T, -1))


class ReluSquaredMLP(nn.Module):
    def __init__(self, c: FrontierConfig):
        super().__init__()
        self.up, self.down = _lin(c.n_embd, 4 * c.n_embd), _lin(4 * c.n_embd, c.n_embd)

    def forward(self, x):
        return self.down(F.relu(self.up(x)).square())


class SiTUGLU(nn.Module):
    """gate = b1 tanh(g / b1) sigmoid(g), up = b2 tanh(u / b2), b1 = 4, b2 = 25; width 8d/3 matches the MLP."""

    def __init__(self, c: FrontierConfig):
        super().__init__()
        inter = round(8 * c.n_embd / 3)
        self.gate, self.up, self.down = _lin(c.n_embd, inter), _lin(c.n_embd, inter), _lin(inter, c.n_embd)

    def forward(self, x):
        g, u = self.gate(x), self.up(x)
        return self.down(4.0 * torch.tanh(g / 4.0) * torch.sigmoid(g) * 25.0 * torch.tanh(u / 25.0))


def _mixer(c: FrontierConfig, layer: int) -> nn.Module:
    v = c.variant
    if v == "qwen_gdn" and (layer + 1) % 4 != 0:
        return GatedDeltaMixer(c, layer)
    if v in ("deepseek_csa", "deepseek_hca"):
        return CompressedAttention(c, layer, heavy=v == "deepseek_hca")
    if v == "glm_mla":
        return MultiLatentAttention(c, layer)
    if v == "motif_gdla":
        return GroupedDifferentialLatentAttention(c, layer)
    return StandardAttention(c, layer)


class AnnealedHyperConnection(nn.Module):
    """n residual streams; read weights sigmoid, write weights 2 sigmoid scaled up from 0 over the first
    ``anneal`` steps, stream mixing matrix made doubly stochastic by Sinkhorn-Knopp in fp32."""

    def __init__(self, c: FrontierConfig):
        super().__init__()
        n = self.n = c.hc_streams
        self.iters, self.anneal = c.hc_sinkhorn_iters, c.hc_anneal_steps
        self.proj = _lin(c.n_embd, 2 * n + n * n)
        self.base = nn.Parameter(torch.cat([torch.zeros(2 * n), torch.eye(n).flatten() * 4.0]))
        self.norm = RMSNorm(c.n_embd)
        self.register_buffer("step", torch.zeros((), dtype=torch.long), persistent=True)

    def forward(self, streams, fn):                                  # streams [B, T, n, C]
        n = self.n
        m = (self.proj(self.norm(streams.mean(2))).float() + self.base.float())
        pre, post, res = m[..., :n].sigmoid(), 2 * m[..., n:2 * n].sigmoid(), m[..., 2 * n:].unflatten(-1, (n, n))
        res = res.exp()
        for _ in range(self.iters):
            res = res / res.sum(-1, keepdim=True)
            res = res / res.sum(-2, keepdim=True)
        scale = min(1.0, (int(self.step) + 1) / self.anneal)
        y = fn((streams.float() * pre.unsqueeze(-1)).sum(2).to(streams.dtype))
        mixed = torch.einsum("btij,btjc->btic", res, streams.float())
        return (mixed + scale * post.unsqueeze(-1) * y.float().unsqueeze(2)).to(streams.dtype)


class FrontierBlock(nn.Module):
    def __init__(self, c: FrontierConfig, layer: int):
        super().__init__()
        zc = c.variant == "zero_centered_rmsnorm"
        self.n1, self.n2 = RMSNorm(c.n_embd, zero_centered=zc), RMSNorm(c.n_embd, zero_centered=zc)
        self.mixer = _mixer(c, layer)
        self.mlp = SiTUGLU(c) if c.variant == "kimi_situ_glu" else ReluSquaredMLP(c)
        self.rconv = ShortConv(c.n_embd, c.sconv_kernel) if c.variant == "inkling_sconv_residual" else None
        self.hc = nn.ModuleList([AnnealedHyperConnection(c), AnnealedHyperConnection(c)]) if c.variant == "motif_mhc" else None

    def forward(self, x, cos, sin):
        if self.hc is not None:
            x = self.hc[0](x, lambda h: self.mixer(self.n1(h), cos, sin))
            return self.hc[1](x, lambda h: self.mlp(self.n2(h)))
        if self.rconv is not None:
            x = self.rconv(x)
        x = x + self.mixer(self.n1(x), cos, sin)
        return x + self.mlp(self.n2(x))


class FrontierLM(nn.Module):
    def __init__(self, config: FrontierConfig):
        super().__init__()
        c = self.config = config
        self.embed = nn.Embedding(c.vocab_size, c.n_embd)
        self.layers = nn.ModuleList(FrontierBlock(c, i) for i in range(c.n_layer))
        self.lm_head = _lin(c.n_embd, c.vocab_size)
        if c.variant == "shared_mtp3":
            self.mtp_mix = _lin(2 * c.n_embd, c.n_embd)
            self.mtp_block = FrontierBlock(FrontierConfig(**{**c.__dict__, "variant": "baseline"}), c.n_layer)

    def init_weights(self, std: float = 0.02):
        for n, p in self.named_parameters():
            if p.dim() >= 2 and not n.endswith(("conv", "bank", ".weight_conv")) and "hc" not in n:
                nn.init.normal_(p, std=std)

    def _logits(self, h):
        return 15.0 * torch.tanh(self.lm_head(rms_norm(h)).float() / 15.0)

    def forward(self, ids, labels=None):
        c = self.config
        B, T = ids.shape
        cos, sin = rope_tables(T, c.head_dim, c.rope_theta, ids.device)
        x = rms_norm(self.embed(ids))
        if c.variant == "motif_mhc":
            x = x.unsqueeze(2).expand(-1, -1, c.hc_streams, -1).contiguous()
        for blk in self.layers:
            x = blk(x, cos, sin)
        if c.variant == "motif_mhc":
            x = x.mean(2)
        logits = self._logits(x)
        if labels is None:
            return logits
        loss = F.cross_entropy(logits.flatten(0, 1), labels.flatten(), ignore_index=-1)
        if c.variant == "shared_mtp3":
            loss = loss + c.mtp_weight * self._mtp(x, ids, labels, cos, sin)
        return loss

    def _mtp(self, hidden, ids, labels, cos, sin):
        """Teacher-forced heads for tokens t+2 .. t+1+depth through ONE shared block."""
        losses, state = [], hidden
        for off in range(1, self.config.mtp_depth + 1):
            valid = ids.size(1) - off
            if valid <= 0:
                break
            teacher = rms_norm(self.embed(ids[:, off:])).to(state.dtype)
            state = self.mtp_block(self.mtp_mix(torch.cat([state[:, :valid], teacher], -1)), cos[:valid], sin[:valid])
            tgt = labels[:, off:]
            losses.append(F.cross_entropy(self._logits(state).flatten(0, 1), tgt.flatten(), ignore_index=-1))
        return torch.stack(losses).mean() if losses else hidden.new_zeros(())


from .protocol import attach_protocol  # noqa: E402  (after the classes it completes)

attach_protocol(FrontierLM)
