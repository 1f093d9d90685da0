"""Qwen3.5-style dense decoder under tensor parallelism with sequence parallelism.

Between tensor-parallel regions every rank holds ``T / TP`` rows of the sequence (embedding, norms,
residual stream, LM head and loss all work on row shards).  QKV and gate/up projections are
column-parallel (their all-gather of rows is fused into the GEMM), attention runs on this rank's heads
over the full sequence, output and down projections are row-parallel (GEMM fused with the
reduce-scatter and the residual add).  Gradients of replicated parameters (norm gains, embedding, LM
head) are summed over the tensor-parallel group by ``sync_replicated_grads``.  One sequence per
micro-batch (the geometry of the Qwen3.5-4B + simplicial configuration: seq 8192, micro-batch 1).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import block_ops
from ..ops import simplicial as sx
from ..ops.attention import causal_attention
from ..parallel import cp as cpar
from ..parallel.tp_layers import ColumnParallelLinear, RowParallelLinear, TPMLP
from .blocks import RMSNorm, apply_rope, rope_tables
from .qwen35 import Qwen35Config


class TPAttention(nn.Module):
    def __init__(self, c: Qwen35Config, simplicial: bool, grp, world: int, group=None, cp=(1, 0, None)):
        super().__init__()
        self.cp_world, self.cp_rank, self.cp_group = cp
        if simplicial and self.cp_world > 1:
            raise ValueError("windowed simplicial layers are not split over the context-parallel group")
        if c.n_heads % world or c.n_kv_heads % world:
            raise ValueError("heads must divide the tensor-parallel size")
        self.c, self.simplicial, self.world = c, simplicial, world
        self.h, self.kv = c.n_heads // world, c.n_kv_heads // world
        width = (c.n_heads + (4 if simplicial else 2) * c.n_kv_heads) * c.head_dim
        self.qkv = ColumnParallelLinear(c.hidden_size, width, grp, world, group)      # this rank's q | k1 | v1 (| k2 | v2) heads
        self.o = RowParallelLinear(c.n_heads * c.head_dim, c.hidden_size, grp, world, group)
        self.q_norm, self.k_norm = RMSNorm(c.head_dim, c.rms_eps), RMSNorm(c.head_dim, c.rms_eps)
        if simplicial:
            self.k2_norm = RMSNorm(c.head_dim, c.rms_eps)

    def forward(self, x_shard, cos, sin, resid):
        c, D = self.c, self.c.head_dim
        y = self.qkv(x_shard)                                       # [T, local width]
        T = y.size(0)
        parts = y.split([self.h * D] + [self.kv * D] * (4 if self.simplicial else 2), -1)
        q = apply_rope(self.q_norm(parts[0].view(1, T, self.h, D)), cos, sin)
        kvs = [p.view(1, T, self.kv, D) for p in parts[1:]]
        k1 = apply_rope(self.k_norm(kvs[0]), cos, sin)
        if self.simplicial:
            k2 = apply_rope(self.k2_norm(kvs[2]), cos, sin)
            o = sx.simplicial_attention(q, k1, k2, kvs[1], kvs[3], c.simplicial_w1, c.simplicial_w2)
        elif self.cp_world > 1:
            o = cpar.cp_causal_attention(q, k1, kvs[1], rank=self.cp_rank, world=self.cp_world, group=self.cp_group)
        else:
            o = causal_attention(q, k1, kvs[1])
        return self.o(o.reshape(T, self.h * D).to(y.dtype), resid)


class TPBlock(nn.Module):
    def __init__(self, c: Qwen35Config, layer: int, grp, world: int, group=None, cp=(1, 0, None)):
        super().__init__()
        self.input_norm, self.post_norm = RMSNorm(c.hidden_size, c.rms_eps), RMSNorm(c.hidden_size, c.rms_eps)
        self.attn = TPAttention(c, c.is_simplicial(layer), grp, world, group, cp)
        self.mlp = TPMLP(c.hidden_size, c.intermediate_size, grp, world, group)

    def forward(self, x, cos, sin):
        x = self.attn(self.input_norm(x), cos, sin, x)              # residual added inside the row-parallel op
        return self.mlp(self.post_norm(x), x)


class Qwen35TP(nn.Module):
    def __init__(self, config: Qwen35Config, grp=None, *, world: int = 1, rank: int = 0, group=None,
                 layer_range: range | None = None, cp=(1, 0, None)):
        """``layer_range`` selects a pipeline stage (embedding on the stage that owns layer 0, final norm
        and LM head on the one that owns the last layer); ``cp`` is (size, rank, group) of the
        context-parallel group."""
        super().__init__()
        c = self.config = config
        self.world, self.rank, self.group = world, rank, group
        self.cp_world, self.cp_rank, self.cp_group = cp
        self.layer_ids = list(layer_range if layer_range is not None else range(c.n_layer))
        self.first, self.last = self.layer_ids[0] == 0, self.layer_ids[-1] == c.n_layer - 1
        if self.first:
            self.embed = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(TPBlock(c, i, grp, world, group, cp) for i in self.layer_ids)
        if self.last:
            self.norm = RMSNorm(c.hidden_size, c.rms_eps)
            self.lm_head = nn.Linear(c.hidden_size, c.vocab_size, bias=False)

    def replicated_parameters(self):
        return [p for p in self.parameters() if not getattr(p, "tensor_model_parallel", False)]

    def sync_replicated_grads(self):
        """Every rank saw different rows: replicated parameters need the sum over the TP group."""
        if self.world == 1:
            return
        for p in self.replicated_parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad, group=self.group)

    @torch.no_grad()
    def load_dense(self, dense) -> None:
        """Shard the weights of a ``Qwen35LM`` (same config) onto this rank."""
        c, W, r, D = self.config, self.world, self.rank, self.config.head_dim
        if self.first:
            self.embed.weight.copy_(dense.embed.weight)
        if self.last:
            self.norm.weight.copy_(dense.norm.weight)
            self.lm_head.weight.copy_(dense.lm_head.weight)
        for mine, ref in zip(self.layers, [dense.layers[i] for i in self.layer_ids]):
            mine.input_norm.weight.copy_(ref.input_norm.weight)
            mine.post_norm.weight.copy_(ref.post_norm.weight)
            simp = mine.attn.simplicial
            widths = [c.n_heads * D] + [c.n_kv_heads * D] * (4 if simp else 2)
            pieces = ref.attn.qkv.weight.split(widths, 0)
            mine.attn.qkv.weight.copy_(torch.cat([p.chunk(W, 0)[r] for p in pieces], 0))
            mine.attn.o.weight.copy_(ref.attn.o.weight.chunk(W, 1)[r])
            for n in ("q_norm", "k_norm") + (("k2_norm",) if simp else ()):
                getattr(mine.attn, n).weight.copy_(getattr(ref.attn, n).weight)
            g, u = ref.gate_up.weight.chunk(2, 0)
            mine.mlp.gate_up.weight.copy_(torch.cat([g.chunk(W, 0)[r], u.chunk(W, 0)[r]], 0))
            mine.mlp.down.weight.copy_(ref.down.weight.chunk(W, 1)[r])

    def local_rows(self, T: int):
        """Absolute positions of this rank's context shard and the row slice of it this TP rank keeps."""
        pos = cpar.shard_positions(T, self.cp_rank, self.cp_world) if self.cp_world > 1 else torch.arange(T)
        rows = pos.numel() // self.world
        return pos, slice(self.rank * rows, (self.rank + 1) * rows)

    def act_shape(self, T: int):
        return (T // self.cp_world // self.world, self.config.hidden_size)

    def forward(self, ids: torch.Tensor, labels: torch.Tensor | None = None, x: torch.Tensor | None = None):
        """ids [1, T] (the same full sequence on every rank of the tensor/context group).

        A first stage embeds its rows; later stages take ``x`` (the previous stage's row shard).  The
        last stage returns its share of the loss: summed over its rows and divided by the global count
        of valid labels, so that the sum over the tensor x context group is the sequence's mean loss.
        Other stages return their output rows."""
        c = self.config
        assert ids.size(0) == 1, "one sequence per micro-batch under sequence parallelism"
        T = ids.size(1)
        pos, sl = self.local_rows(T)
        pos = pos.to(ids.device)
        dt = torch.bfloat16 if ids.device.type == "cuda" else torch.float32
        if self.first:
            x = self.embed(ids[0, pos[sl]]).to(dt)
        cos, sin = rope_tables(T, c.head_dim, c.rope_theta, ids.device)
        cos, sin = cos[pos], sin[pos]
        for blk in self.layers:
            x = blk(x, cos, sin)
        if not self.last:
            return x
        logits = self.lm_head(self.norm(x).to(self.lm_head.weight.dtype))
        if labels is None:
            return logits.float()
        loss_sum = block_ops.cross_entropy_sum(logits, labels[0, pos[sl]])
        return loss_sum / labels.ne(-1).sum().clamp_min(1)
