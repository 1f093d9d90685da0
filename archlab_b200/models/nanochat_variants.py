"""nanochat-sized families that add one mechanism to the speedrun GPT trunk.

* ``EngramGPT``: suffix n-gram memories (``blocks.EngramMemory``) read before chosen layers; token ids
  pass through a token map (identity by default, replaceable by a tokenizer-derived compression map)
  before hashing.  Reference wiring: src/archlab/architectures/base.py:491-518, 919-931.
* ``MhcGPT``: every sublayer sits inside a manifold-constrained hyper-connection over ``n`` residual
  streams (``blocks.HyperConnection``): the sublayer reads a gated sum of the streams, its output is
  written back to every stream and the streams are mixed by a Sinkhorn-normalised matrix; the streams
  are averaged after the last layer.  Reference wiring: base.py:519-527, 911-947, 973-976.

Both keep the trunk's per-layer residual / embedding gains, value embeddings, smear gate and mid-depth
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
