"""Qwen3.8-style hybrid language models: gated delta-net (GDN) token mixers with one gated full
GQA layer every ``full_attention_interval`` layers, SwiGLU or sparse-MoE feed-forward, optional
top-k sparse attention (token indexer), optional hashed n-gram per-layer embedding, and a
multi-token-prediction (MTP) head.

Covers the dense 27B text family (quarter / full geometry) and the Flash-Next MoE family
(src/archlab/architectures/qwen38_27b.py:29-590, qwen38_flash_next.py:19-1319).  The delta rule
runs through ``ops.delta_rule`` (chunk-parallel form), routing through ``models.moe``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, replace

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.attention import causal_attention
from ..ops import delta_rule
from . import moe
from .blocks import NgramHash, OwnerShardedEmbedding, RMSNorm, apply_rope, rope_tables


@dataclass(frozen=True)
class Qwen38Config:
    vocab_size: int = 248_320
    sequence_len: int = 2048
    eos_token_id: int = 248_044
    num_hidden_layers: int = 16
    hidden_size: int = 1280
    intermediate_size: int = 4352
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7
    partial_rotary_factor: float = 0.25
    full_attention_interval: int = 4
    attention_heads: int = 6
    attention_kv_heads: int = 1
    attention_head_dim: int = 64
    linear_qk_heads: int = 4
    linear_v_heads: int = 12
    linear_key_dim: int = 32
    linear_value_dim: int = 32
    linear_conv_kernel: int = 4
    mtp_layers: int = 1
    mtp_loss_weight: float = 0.1
    mtp_fusion: bool = False
    # Flash-Next additions (0 experts = dense SwiGLU)
    n_experts: int = 0
    experts_top_k: int = 3
    moe_intermediate_size: int = 512
    shared_expert_gated: bool = True
    router_score: str = "softmax"
    router_aux_weight: float = 1e-3
    router_z_weight: float = 1e-4
    sparse_top_k: int = 0                 # > 0: full-attention layers attend to the indexer's top-k tokens
    indexer_heads: int = 4
    indexer_dim: int = 32
    ngram_size: int = 0                   # > 0: hashed n-gram per-layer embedding added to the input
    ngram_heads_per_order: int = 2
    ngram_head_vocab: int = 4099
    ngram_dim: int = 64
    arch_family: str = "qwen38_27b_quarter_text"

    @classmethod
    def for_scale(cls, scale: str, **overrides) -> "Qwen38Config":
        if scale == "quarter":
            return replace(cls(), **overrides)
        if scale == "full":
            values = dict(num_hidden_layers=64, hidden_size=5120, intermediate_size=17408, attention_heads=24,
                          attention_kv_heads=4, attention_head_dim=256, linear_qk_heads=16, linear_v_heads=48,
                          linear_key_dim=128, linear_value_dim=128, mtp_fusion=True, arch_family="qwen38_27b_text")
        elif scale == "flash_next_quarter":
            values = dict(n_experts=128, experts_top_k=3, moe_intermediate_size=192, sparse_top_k=256, ngram_size=3,
                          arch_family="qwen38_flash_next_quarter")
        elif scale == "tiny":
            values = dict(vocab_size=512, eos_token_id=0, sequence_len=64, num_hidden_layers=4, hidden_size=64,
                          intermediate_size=128, attention_heads=4, attention_kv_heads=2, attention_head_dim=16,
                          linear_qk_heads=2, linear_v_heads=4, linear_key_dim=16, linear_value_dim=16,
                          arch_family="qwen38_tiny")
        else:
            raise ValueError(f"unsupported Qwen3.8 scale: {scale}")
        values.update(overrides)
        return replace(cls(), **values)

    def __post_init__(self):
        if self.attention_heads % self.attention_kv_heads:
            raise ValueError("attention KV heads must divide query heads")
        if self.linear_v_heads % self.linear_qk_heads:
            raise ValueError("linear QK heads must divide value heads")
        rot = int(self.attention_head_dim * self.partial_rotary_factor)
        if rot < 2 or rot % 2:
            raise ValueError("partial RoPE must retain a positive even dimension")
        if self.mtp_layers not in (0, 1):
            raise ValueError("at most one MTP layer is supported")

    def to_dict(self) -> dict:
        return asdict(self)


def _lin(i: int, o: int) -> nn.Linear:
    return nn.Linear(i, o, bias=False)


class GatedDeltaNet(nn.Module):
    """Fused q/k/v projection -> causal depthwise conv + SiLU -> delta rule with scalar decay
    ``-exp(a_log) softplus(logit + dt_bias)`` and ``beta = sigmoid`` -> per-head RMSNorm ->
    SiLU(z) output gate -> projection."""

    def __init__(self, c: Qwen38Config):
        super().__init__()
        self.qh, self.vh, self.kd, self.vd = c.linear_qk_heads, c.linear_v_heads, c.linear_key_dim, c.linear_value_dim
        qw, vw = self.qh * self.kd, self.vh * self.vd
        self.qkv = _lin(c.hidden_size, 2 * qw + vw)
        self.z = _lin(c.hidden_size, vw)
        self.ba = _lin(c.hidden_size, 2 * self.vh)
        self.conv_weight = nn.Parameter(torch.empty(2 * qw + vw, c.linear_conv_kernel))
        self.a_log = nn.Parameter(torch.zeros(self.vh))
        self.dt_bias = nn.Parameter(torch.full((self.vh,), -4.0))
        self.output_norm = RMSNorm(self.vd, c.rms_norm_eps)
        self.out = _lin(vw, c.hidden_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, _ = x.shape
        qw, vw = self.qh * self.kd, self.vh * self.vd
        qkv = delta_rule.causal_conv1d(self.qkv(x), self.conv_weight)
        q, k, v = qkv.split((qw, qw, vw), -1)
        b_logit, d_logit = self.ba(x).chunk(2, -1)
        decay = -self.a_log.float().exp() * F.softplus(d_logit.float() + self.dt_bias.float())
        rep = self.vh // self.qh
        q = q.view(B, T, self.qh, self.kd).repeat_interleave(rep, 2)
        k = k.view(B, T, self.qh, self.kd).repeat_interleave(rep, 2)
        o = delta_rule.gated_delta_rule(q, k, v.view(B, T, self.vh, self.vd), decay, b_logit.sigmoid())
        o = self.output_norm(o.to(x.dtype)) * F.silu(self.z(x).view(B, T, self.vh, self.vd))
        return self.out(o.flatten(-2))


class TokenIndexer(nn.Module):
    """Lightweight multi-head scorer choosing which past tokens a sparse-attention query reads:
    score(t, s) = sum_h w_h(t) relu(q_h(t) . k(s)), causal, top-k per query."""

    def __init__(self, c: Qwen38Config):
        super().__init__()
        self.h, self.d, self.top_k = c.indexer_heads, c.indexer_dim, c.sparse_top_k
        self.q = _lin(c.hidden_size, self.h * self.d)
        self.k = _lin(c.hidden_size, self.d)
        self.w = _lin(c.hidden_size, self.h)

    def scores(self, x: torch.Tensor) -> torch.Tensor:
        B, T, _ = x.shape
        q = self.q(x).view(B, T, self.h, self.d).float()
        k = self.k(x).float()
        s = torch.einsum("bthd,bsd->bhts", q, k).relu() * self.d ** -0.5
        s = (s * self.w(x).float().transpose(1, 2).unsqueeze(-1)).sum(1)              # [B, T, T]
        causal = torch.ones(T, T, dtype=torch.bool, device=x.device).tril()
        return s.masked_fill(~causal, float("-inf"))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """-> boolean mask [B, T, T] of the selected (causal) keys."""
        s = self.scores(x)
        T = s.size(-1)
        k = min(self.top_k, T)
        idx = s.topk(k, -1).indices
        mask = torch.zeros_like(s, dtype=torch.bool).scatter_(-1, idx, True)
        return mask & torch.isfinite(s)


class GatedAttention(nn.Module):
    """GQA with the sigmoid output gate fused into the q projection, per-head q/k RMSNorm and
    partial rotary embedding; optionally restricted to the indexer's top-k keys."""

    def __init__(self, c: Qwen38Config):
        super().__init__()
        self.h, self.kv, self.d = c.attention_heads, c.attention_kv_heads, c.attention_head_dim
        self.rot = int(self.d * c.partial_rotary_factor)
        self.q_gate = _lin(c.hidden_size, 2 * self.h * self.d)
        self.k = _lin(c.hidden_size, self.kv * self.d)
        self.v = _lin(c.hidden_size, self.kv * self.d)
        self.q_norm = RMSNorm(self.d, c.rms_norm_eps)
        self.k_norm = RMSNorm(self.d, c.rms_norm_eps)
        self.out = _lin(self.h * self.d, c.hidden_size)
        self.indexer = TokenIndexer(c) if c.sparse_top_k > 0 else None

    def forward(self, x, cos, sin):
        B, T, _ = x.shape
        q, gate = self.q_gate(x).view(B, T, self.h, 2 * self.d).chunk(2, -1)
        k = self.k(x).view(B, T, self.kv, self.d)
        v = self.v(x).view(B, T, self.kv, self.d)
        q = apply_rope(self.q_norm(q), cos, sin, rot_dim=self.rot)
        k = apply_rope(self.k_norm(k), cos, sin, rot_dim=self.rot)
        if self.indexer is not None and T > self.indexer.top_k:
            rep = self.h // self.kv
            k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
            mask = self.indexer(x.detach()).unsqueeze(1)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask).transpose(1, 2)
        else:
            o = causal_attention(q, k, v)
        o = o * torch.sigmoid(gate)
        return self.out(o.reshape(B, T, self.h * self.d))


class DenseMLP(nn.Module):
    def __init__(self, c: Qwen38Config):
        super().__init__()
        self.gate, self.up = _lin(c.hidden_size, c.intermediate_size), _lin(c.hidden_size, c.intermediate_size)
        self.down = _lin(c.intermediate_size, c.hidden_size)

    def forward(self, x):
        return self.down(F.silu(self.gate(x)) * self.up(x))


class HybridBlock(nn.Module):
    def __init__(self, c: Qwen38Config, layer_idx: int, *, force_full: bool = False):
        super().__init__()
        self.input_norm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.mlp_norm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        full = force_full or (layer_idx + 1) % c.full_attention_interval == 0
        self.attention_kind = "full_attention" if full else "gdn"
        self.attention = GatedAttention(c) if full else GatedDeltaNet(c)
        if c.n_experts > 0:
            self.mlp = moe.SparseMoE(c.hidden_size, c.moe_intermediate_size, c.n_experts, c.experts_top_k, n_shared=1,
                                     score=c.router_score, gated_shared=c.shared_expert_gated)
        else:
            self.mlp = DenseMLP(c)

    def forward(self, x, cos, sin):
        h = self.input_norm(x)
        x = x + (self.attention(h, cos, sin) if self.attention_kind == "full_attention" else self.attention(h))
        return x + self.mlp(self.mlp_norm(x))


class MTPHead(nn.Module):
    """Predicts token t+2 from [norm(hidden_t), norm(embedding_{t+1})] through one full-attention block."""

    def __init__(self, c: Qwen38Config):
        super().__init__()
        self.fusion = c.mtp_fusion
        if self.fusion:
            self.norm_embedding = RMSNorm(c.hidden_size, c.rms_norm_eps)
            self.norm_hidden = RMSNorm(c.hidden_size, c.rms_norm_eps)
            self.fc = _lin(2 * c.hidden_size, c.hidden_size)
        self.block = HybridBlock(c, c.num_hidden_layers, force_full=True)
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps)

    def forward(self, hidden, shifted_embedding, cos, sin):
        if self.fusion:
            x = self.fc(torch.cat([self.norm_hidden(hidden), self.norm_embedding(shifted_embedding)], -1))
        else:
            x = hidden + shifted_embedding
        return self.norm(self.block(x, cos, sin))


class Qwen38LM(nn.Module):
    def __init__(self, config: Qwen38Config, *, ple_owner_rank: int = 0, ple_owners: int = 1, ple_group=None):
        super().__init__()
        c = self.config = config
        self.token_embedding = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(HybridBlock(c, i) for i in range(c.num_hidden_layers))
        self.final_norm = RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.lm_head = _lin(c.hidden_size, c.vocab_size)
        self.mtp = MTPHead(c) if c.mtp_layers else None
        if c.ngram_size > 1:
            heads = (c.ngram_size - 1) * c.ngram_heads_per_order
            self.ple_hash = NgramHash(c.vocab_size, c.ngram_size, c.ngram_heads_per_order, [c.ngram_head_vocab] * heads,
                                      c.eos_token_id)
            parts = max(ple_owners, 1)
            rows = -(-heads * c.ngram_head_vocab // parts)
            self.ple_table = OwnerShardedEmbedding(parts, rows, c.ngram_dim, owner_rank=ple_owner_rank, owners=ple_owners,
                                                   group=ple_group)
            self.ple_proj = _lin(heads * c.ngram_dim, c.hidden_size)
        else:
            self.ple_hash = None
        self.last_loss_metrics: dict = {}
        self._tag()

    # --- optimizer tagging: matrices of the mixers / MLPs go to Muon, everything else to AdamW
    def _tag(self):
        for p in self.parameters():
            p.archlab_optimizer, p.archlab_optimizer_category = "adamw", "scalar_norm_or_non_linear"
        for p in self.token_embedding.parameters():
            p.archlab_optimizer_category = "input_embedding"
        for p in self.lm_head.parameters():
            p.archlab_optimizer_category = "output_head"
        blocks = list(self.layers) + ([self.mtp.block] if self.mtp is not None else [])
        for blk in blocks:
            att = blk.attention
            names = ("qkv", "out") if isinstance(att, GatedDeltaNet) else ("q_gate", "k", "v", "out")
            # logical Muon matrices of the fused projections (src/archlab/architectures/qwen38_flash_next.py:995-1029):
            # the GDN q/k/v projection per head (key_dim rows each), the gated attention query per head
            split = {"qkv": att.kd} if isinstance(att, GatedDeltaNet) else {"q_gate": att.d}
            for n in names:
                w = getattr(att, n).weight
                w.archlab_optimizer, w.archlab_optimizer_category = "muon", f"{blk.attention_kind}_{n}"
                rows = split.get(n)
                if rows and w.shape[0] % rows == 0:
                    w.archlab_muon_split_rows = rows
            if isinstance(blk.mlp, DenseMLP):
                for n in ("gate", "up", "down"):
                    w = getattr(blk.mlp, n).weight
                    w.archlab_optimizer, w.archlab_optimizer_category = "muon", f"mlp_{n}"
            else:
                for n, w in (("experts_gate_up", blk.mlp.experts.gate_up), ("experts_down", blk.mlp.experts.down)):
                    w.archlab_optimizer, w.archlab_optimizer_category = "muon", n
                blk.mlp.experts.gate_up.archlab_muon_split_rows = blk.mlp.experts.gate_up.shape[-2] // 2   # gate / up halves
        if self.mtp is not None and self.mtp.fusion:
            self.mtp.fc.weight.archlab_optimizer = "muon"
            self.mtp.fc.weight.archlab_optimizer_category = "mtp_fusion"

    def optimizer_contract(self) -> dict:
        out: dict = {}
        for _, p in self.named_parameters():
            b = out.setdefault(p.archlab_optimizer, {"tensors": 0, "parameters": 0, "logical_matrices": 0})
            b["tensors"] += 1
            b["parameters"] += p.numel()
            b["logical_matrices"] += (p.shape[0] if p.ndim == 3 else 1) if p.archlab_optimizer == "muon" else 0
        return {"optimizers": out, "all_trainable_parameters_assigned_once": True, "frozen_parameters": 0}

    @torch.no_grad()
    def init_weights(self, std: float = 0.02):
        for name, p in self.named_parameters():
            if p.ndim >= 2:
                nn.init.normal_(p, std=std)
        for m in self.modules():
            if isinstance(m, RMSNorm):
                m.weight.fill_(0.0 if m.zero_centered else 1.0)
            if isinstance(m, GatedDeltaNet):
                m.a_log.copy_(torch.empty_like(m.a_log).uniform_(0.01, 16.0).log())
                m.dt_bias.fill_(1.0)
            if isinstance(m, OwnerShardedEmbedding):
                m.reset_parameters(std)
            if isinstance(m, moe.SparseMoE) and m.shared_gate is not None:
                m.shared_gate.weight.zero_()

    def num_scaling_params(self) -> dict:
        emb = self.token_embedding.weight.numel() + self.lm_head.weight.numel()
        mtp = sum(p.numel() for p in self.mtp.parameters()) if self.mtp is not None else 0
        total = sum(p.numel() for p in self.parameters())
        return {"embeddings_and_head": emb, "text_backbone": total - emb - mtp, "mtp": mtp, "total": total}

    def estimate_flops(self) -> float:
        return 6.0 * float(self.num_scaling_params()["total"])

    def routers(self):
        return [b.mlp for b in self.layers if isinstance(b.mlp, moe.SparseMoE)]

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, *, loss_reduction: str = "mean"):
        if input_ids.ndim != 2:
            raise ValueError("input_ids must have shape [batch, sequence]")
        c = self.config
        B, T = input_ids.shape
        dt = torch.bfloat16 if input_ids.device.type == "cuda" else torch.float32
        x = self.token_embedding(input_ids).to(dt)
        if self.ple_hash is not None:
            x = x + self.ple_proj(self.ple_table(self.ple_hash(input_ids)).flatten(-2).to(dt))
        cos, sin = rope_tables(T, int(c.attention_head_dim * c.partial_rotary_factor), c.rope_theta, input_ids.device)
        with torch.autocast(input_ids.device.type, dtype=dt, enabled=dt != torch.float32):
            for layer in self.layers:
                x = layer(x, cos, sin)
            hidden = self.final_norm(x)
            logits = self.lm_head(hidden).float()
            if labels is None:
                return logits
            ce = F.cross_entropy(logits.flatten(0, 1), labels.flatten(), ignore_index=-1, reduction="none").view_as(labels)
            extra = torch.zeros_like(ce)
            if self.mtp is not None and T > 1:
                emb = self.token_embedding(input_ids[:, 1:]).to(hidden.dtype)
                h2 = self.mtp(hidden[:, :-1], emb, cos[:-1], sin[:-1])
                l2 = F.cross_entropy(self.lm_head(h2).float().flatten(0, 1), labels[:, 1:].flatten(), ignore_index=-1,
                                     reduction="none").view(B, T - 1)
                extra = torch.cat([c.mtp_loss_weight * l2, extra[:, -1:]], 1)
        valid = labels.ne(-1)
        n = valid.sum().clamp_min(1)
        losses = ce + extra
        self.last_loss_metrics = {"cross entropy": (ce * valid).sum().detach() / n, "mtp loss": (extra * valid).sum().detach() / n}
        aux = sum((m.last_metrics["aux_loss"] for m in self.routers()), start=torch.zeros((), device=ce.device))
        if loss_reduction == "none":
            return losses
        total = losses.sum() if loss_reduction == "sum" else losses.sum() / n
        if loss_reduction not in ("sum", "mean"):
            raise ValueError(f"unsupported loss reduction: {loss_reduction}")
        return total + c.router_aux_weight * aux if self.routers() else total


from .protocol import attach_protocol  # noqa: E402  (after the classes it completes)

attach_protocol(Qwen38LM)
