"""nanochat-sized families that add one mechanism to the speedrun GPT trunk.

* ``EngramGPT``: suffix n-gram memories (``blocks.EngramMemory``) read before chosen layers; token ids
  pass through a token map (identity by default, replaceable by a tokenizer-derived compression map)
  before hashing.  Reference wiring: src/archlab/architectures/base.py:491-518, 919-931.
* ``MhcGPT``: every sublayer sits inside a manifold-constrained hyper-connection over ``n`` residual
  streams (``blocks.HyperConnection``): the sublayer reads a gated sum of the streams, its output is
  written back to every stream and the streams are mixed by a Sinkhorn-normalised matrix; the streams
  are averaged after the last layer.  Reference wiring: base.py:519-527, 911-947, 973-976.

* ``DsaGPT``: lightning-indexer top-k sparse attention with a dense indexer warm-up stage (further down).

All keep the trunk's per-layer residual / embedding gains, value embeddings, smear gate and mid-depth
back-out exactly as ``nanochat.GPT`` applies them, so the baseline is recovered when the mechanism's
output is zero.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .blocks import EngramMemory, HyperConnection, rms_norm
from .nanochat import GPT, GPTConfig


@dataclass
class EngramGPTConfig(GPTConfig):
    engram_layers: tuple[int, ...] = (2,)
    engram_ngram_orders: tuple[int, ...] = (2, 3)
    engram_num_heads: int = 8
    engram_dim: int = 0                      # 0: half the model width
    engram_vocab_multiplier: int = 5
    engram_kernel_size: int = 4
    engram_seed: int = 0


class EngramGPT(GPT):
    def __init__(self, config: EngramGPTConfig):
        super().__init__(config)
        layers = tuple(config.engram_layers)
        if not layers:
            raise ValueError("the Engram family needs at least one memory layer")
        if any(l < 0 or l >= config.n_layer for l in layers) or len(set(layers)) != len(layers):
            raise ValueError(f"Engram layers {layers} are invalid for depth {config.n_layer}")
        dim = config.engram_dim or config.n_embd // 2
        self.engrams = nn.ModuleDict({
            str(l): EngramMemory(hidden=config.n_embd, memory_dim=dim, vocab=config.vocab_size,
                                 vocab_multiplier=config.engram_vocab_multiplier, heads=config.engram_num_heads,
                                 orders=tuple(config.engram_ngram_orders), layer_idx=l, seed=config.engram_seed,
                                 kernel=config.engram_kernel_size)
            for l in layers})
        self.register_buffer("engram_token_map", torch.arange(config.vocab_size), persistent=True)
        self.register_buffer("engram_pad_id", torch.zeros((), dtype=torch.long), persistent=True)

    @torch.no_grad()
    def init_weights(self) -> None:
        super().init_weights()
        for mem in self.engrams.values():
            nn.init.normal_(mem.embedding.weight, std=0.02)
            nn.init.normal_(mem.key_proj.weight, std=mem.key_proj.in_features ** -0.5)
            nn.init.zeros_(mem.value_proj.weight)             # the memory starts silent: the baseline trunk
            for p in mem.short_conv.parameters():
                if p.dim() > 1:
                    nn.init.normal_(p, std=0.02)
        self.engram_token_map.copy_(torch.arange(self.config.vocab_size, device=self.engram_token_map.device))
        self.engram_pad_id.zero_()

    def configure_engram_token_map(self, token_map: torch.Tensor, pad_id: int) -> None:
        """``token_map[v]`` = the id hashed in place of token ``v`` (e.g. case- and whitespace-folded)."""
        if token_map.shape != self.engram_token_map.shape:
            raise ValueError(f"expected token map shape {tuple(self.engram_token_map.shape)}, got {tuple(token_map.shape)}")
        self.engram_token_map.copy_(token_map.to(self.engram_token_map.device, torch.long))
        self.engram_pad_id.copy_(self.engram_token_map[int(pad_id)])

    def trunk(self, idx: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        T = idx.size(1)
        cos, sin = self.cos[:T], self.sin[:T]
        x = self.embed(idx)
        x0, x_backout = x, None
        hashed = self.engram_token_map[idx]
        pad = int(self.engram_pad_id)
        for i, block in enumerate(self.transformer.h):
            x = self.resid_lambdas[i].to(x.dtype) * x + self.x0_lambdas[i].to(x.dtype) * x0
            if str(i) in self.engrams:
                x = x + self.engrams[str(i)](x, hashed, pad)
            ve = self.value_embeds[str(i)](idx).to(x.dtype) if str(i) in self.value_embeds else None
            x = block(x, ve, cos, sin, self.window_sizes[i])
            if i == cfg.n_layer // 2:
                x_backout = x
        if x_backout is not None:
            x = x - self.backout_lambda.to(x.dtype) * x_backout
        return rms_norm(x)


@dataclass
class MhcGPTConfig(GPTConfig):
    mhc_num_streams: int = 4
    mhc_init_gating_factor: float = 0.01
    mhc_sinkhorn_iterations: int = 20


class MhcGPT(GPT):
    def __init__(self, config: MhcGPTConfig):
        super().__init__(config)
        self.mhc_connections = nn.ModuleList(
            HyperConnection(config.n_embd, config.mhc_num_streams, config.mhc_sinkhorn_iterations,
                            config.mhc_init_gating_factor) for _ in range(2 * config.n_layer))

    @torch.no_grad()
    def init_weights(self) -> None:
        super().init_weights()
        for c in self.mhc_connections:
            c.init_weights()

    def trunk(self, idx: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        B, T = idx.shape
        cos, sin = self.cos[:T], self.sin[:T]
        x = self.embed(idx).unsqueeze(-2).expand(B, T, cfg.mhc_num_streams, cfg.n_embd).contiguous()
        x0, x_backout = x, None
        for i, block in enumerate(self.transformer.h):
            x = self.resid_lambdas[i].to(x.dtype) * x + self.x0_lambdas[i].to(x.dtype) * x0
            ve = self.value_embeds[str(i)](idx).to(x.dtype) if str(i) in self.value_embeds else None
            conn = self.mhc_connections[2 * i]
            inp, post, res = conn.prepare(x)
            x = conn.combine(x, block.attn(rms_norm(inp), ve, cos, sin, self.window_sizes[i]), post, res)
            conn = self.mhc_connections[2 * i + 1]
            inp, post, res = conn.prepare(x)
            x = conn.combine(x, block.mlp(rms_norm(inp)), post, res)
            if i == cfg.n_layer // 2:
                x_backout = x
        x = x.mean(-2)
        if x_backout is not None:
            x = x - self.backout_lambda.to(x.dtype) * x_backout.mean(-2)
        return rms_norm(x)


# ------------------------------------------------------------------------------------------------
# DeepSeek sparse attention at nanochat size
# ------------------------------------------------------------------------------------------------
@dataclass
class DsaGPTConfig(GPTConfig):
    dsa_top_k: int = 32
    dsa_index_heads: int = 2
    dsa_index_head_dim: int = 32
    dsa_index_rope_dim: int = 8
    dsa_query_chunk_size: int = 128          # kept for checkpoints of the chunked backend; the masked form ignores it
    dsa_backend: str = "sdpa_masked"
    dsa_warmup_indexer_lr: float = 1e-3
    dsa_sparse_indexer_lr: float = 7.3e-6


class DsaSelfAttention(nn.Module):
    """nanochat attention whose keys are chosen per query by a lightning indexer (ReLU dot products of a few small
    heads, weighted per head; src/archlab/architectures/dsa.py:85-233).  Two stages: ``dense`` runs the ordinary causal
    attention and trains only the indexer towards the head-averaged attention distribution (KL over all causal keys);
    ``sparse`` attends to the top-k keys and keeps aligning the indexer on the selected set.  The indexer reads a
    detached copy of the hidden state, so the language-model loss never reaches it."""

    def __init__(self, config: DsaGPTConfig, layer_idx: int):
        super().__init__()
        from .nanochat import CausalSelfAttention

        self.inner = CausalSelfAttention(config, layer_idx)
        self.config = config
        Hi, Di = config.dsa_index_heads, config.dsa_index_head_dim
        self.index_q = nn.Linear(config.n_embd, Hi * Di, bias=False)
        self.index_k = nn.Linear(config.n_embd, Di, bias=False)
        self.index_w = nn.Linear(config.n_embd, Hi, bias=False)
        self.dense = True
        self.last_kl = None

    def forward(self, x, ve, cos, sin, window):
        import torch.nn.functional as F

        from ..ops import dsa
        from .blocks import apply_rope, rope_tables
        from .nanochat import sdpa_window

        a, cfg = self.inner, self.config
        B, T, _ = x.shape
        q = a.c_q(x).view(B, T, cfg.n_head, cfg.head_dim)
        k = a.c_k(x).view(B, T, cfg.n_kv_head, cfg.head_dim)
        v = a.c_v(x).view(B, T, cfg.n_kv_head, cfg.head_dim)
        if ve is not None:
            v = v + (3 * torch.sigmoid(a.ve_gate(x[..., : a.ve_gate_channels]))).unsqueeze(-1) * ve.view_as(v)
        q, k = rms_norm(apply_rope(q, cos, sin)) * 1.2, rms_norm(apply_rope(k, cos, sin)) * 1.2
        # indexer on a detached input
        xd = x.detach()
        Hi, Di, R = cfg.dsa_index_heads, cfg.dsa_index_head_dim, cfg.dsa_index_rope_dim
        ic, isn = rope_tables(T, R, 10000.0, x.device)
        iq = apply_rope(self.index_q(xd).view(B, T, Hi, Di), ic.to(x.dtype), isn.to(x.dtype), rot_dim=R)
        ik = apply_rope(self.index_k(xd).view(B, T, 1, Di), ic.to(x.dtype), isn.to(x.dtype), rot_dim=R).squeeze(2)
        scores = dsa.indexer_scores(iq, ik, self.index_w(xd) * Hi ** -0.5)                 # [B, T, T], -inf above the diagonal
        causal = torch.isfinite(scores)
        if self.dense:
            y = sdpa_window(q, k, v, window)
            valid = causal
        else:
            kth = scores.topk(min(cfg.dsa_top_k, T), dim=-1).values[..., -1:]
            valid = causal & (scores >= kth)
            rep = cfg.n_head // cfg.n_kv_head
            kk, vv = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
            y = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                               attn_mask=valid.unsqueeze(1)).transpose(1, 2)
        if self.training:
            with torch.no_grad():                                                        # head-averaged attention target
                rep = cfg.n_head // cfg.n_kv_head
                s = torch.einsum("bshd,bkhd->bhsk", q.float(), k.repeat_interleave(rep, 2).float()) * cfg.head_dim ** -0.5
                target = s.masked_fill(~causal.unsqueeze(1), float("-inf")).softmax(-1).mean(1)
            self.last_kl = dsa.indexer_kl(target, scores, valid)
        return a.c_proj(y.contiguous().view(B, T, -1))


class DsaGPT(GPT):
    def __init__(self, config: DsaGPTConfig):
        super().__init__(config)
        if config.dsa_backend != "sdpa_masked":
            raise ValueError("this build runs the masked-attention form of the sparse stage")
        for i, block in enumerate(self.transformer.h):
            block.attn = DsaSelfAttention(config, i)

    @torch.no_grad()
    def init_weights(self) -> None:
        # the trunk initialiser addresses block.attn.c_q ... directly: expose the wrapped projections under those names
        wrapped = [b.attn for b in self.transformer.h]
        for b in self.transformer.h:
            b.attn = b.attn.inner
        try:
            super().init_weights()
        finally:
            for b, w in zip(self.transformer.h, wrapped):
                b.attn = w
        for w in wrapped:
            for lin in (w.index_q, w.index_k, w.index_w):
                nn.init.normal_(lin.weight, std=lin.in_features ** -0.5)

    def set_stage(self, stage: str) -> None:
        """``dense``: indexer warm-up under full attention; ``sparse``: top-k attention."""
        if stage not in ("dense", "sparse"):
            raise ValueError("stage must be dense or sparse")
        for b in self.transformer.h:
            b.attn.dense = stage == "dense"

    def indexer_parameters(self):
        return [p for b in self.transformer.h for lin in (b.attn.index_q, b.attn.index_k, b.attn.index_w) for p in lin.parameters()]

    def forward(self, idx, targets=None, loss_reduction: str = "mean"):
        out = super().forward(idx, targets, loss_reduction)
        if targets is None or not self.training or loss_reduction != "mean":
            return out
        kls = [b.attn.last_kl for b in self.transformer.h if b.attn.last_kl is not None]
        return out + torch.stack(kls).sum() if kls else out
