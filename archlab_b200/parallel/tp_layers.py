"""Tensor-parallel linear layers under sequence parallelism, built on the fused GEMM + collective
kernels of ``parallel.tp``.

Activations between tensor-parallel regions are sharded over the sequence (rows).
``ColumnParallelLinear``: all-gather(rows) fused into the GEMM; output keeps all rows, 1/TP of the
columns.  ``RowParallelLinear``: GEMM fused with the reduce-scatter; output is this rank's rows, all
columns.  Each backward is the other's pattern (input gradient) plus one local tcgen05 GEMM (weight
gradient) - the role of Megatron's TEColumnParallelLinear / TERowParallelLinear
(src/archlab/megatron/qwen38_flash_next_model.py:179-205).  Off the GPU the decomposed reference
functions run instead, so the same module trains under gloo in tests.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import block_ops
from ..ops import gemm as G
from . import tp as T


class _ColumnParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, grp):
        y = T.ag_gemm(grp, x_shard, w)
        xg = grp.gathered_view(x_shard.size(1)).clone()          # the shared gather buffer is reused by later layers
        ctx.save_for_backward(xg, w)
        ctx.grp = grp
        return y

    @staticmethod
    def backward(ctx, gy):
        xg, w = ctx.saved_tensors
        gy = gy.contiguous()
        gx = T.gemm_rs(ctx.grp, gy, w, w_mn=True)                # (dY @ W) reduce-scattered over rows
        gw = G.gemm(gy, xg, a_mn=True, b_mn=True)                # dY^T @ gather(X)
        return gx, gw, None


class _RowParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, resid, grp):
        ctx.save_for_backward(a, w)
        ctx.grp, ctx.has_resid = grp, resid is not None
        return T.gemm_rs(grp, a.contiguous(), w, resid=resid)

    @staticmethod
    def backward(ctx, gout):
        a, w = ctx.saved_tensors
        gout = gout.contiguous()
        ga = T.ag_gemm(ctx.grp, gout, w, w_mn=True)              # gather(dOut) @ W
        gg = ctx.grp.gathered_view(gout.size(1))
        gw = G.gemm(gg, a, a_mn=True, b_mn=True)                 # gather(dOut)^T @ A
        return ga, gw, (gout if ctx.has_resid else None), None


def _fused_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


class ColumnParallelLinear(nn.Module):
    """weight [out_features / TP, in_features]; input [rows_per_rank, in] -> output [TP * rows_per_rank, out / TP]."""

    def __init__(self, in_features: int, out_features: int, grp: T.TPGroup | None, world: int, group=None):
        super().__init__()
        if out_features % world:
            raise ValueError("output features must divide the tensor-parallel size")
        self.grp, self.world, self.group = grp, world, group
        self.weight = nn.Parameter(torch.empty(out_features // world, in_features))
        self.weight.tensor_model_parallel, self.weight.partition_dim = True, 0

    def forward(self, x_shard):
        if _fused_ok(x_shard) and self.grp is not None:
            return _ColumnParallel.apply(x_shard, self.weight.to(x_shard.dtype), self.grp)
        return _gather_rows(x_shard, self.group) @ self.weight.to(x_shard.dtype).t()


class RowParallelLinear(nn.Module):
    """weight [out_features, in_features / TP]; input [TP * rows_per_rank, in / TP] -> output [rows_per_rank, out]."""

    def __init__(self, in_features: int, out_features: int, grp: T.TPGroup | None, world: int, group=None):
        super().__init__()
        if in_features % world:
            raise ValueError("input features must divide the tensor-parallel size")
        self.grp, self.world, self.group = grp, world, group
        self.weight = nn.Parameter(torch.empty(out_features, in_features // world))
        self.weight.tensor_model_parallel, self.weight.partition_dim = True, 1

    def forward(self, a, resid=None):
        if _fused_ok(a) and self.grp is not None:
            return _RowParallel.apply(a, self.weight.to(a.dtype), resid, self.grp)
        y = _reduce_scatter_rows(a @ self.weight.to(a.dtype).t(), self.group)
        return y if resid is None else y + resid


# ------------------------------------------------------------------------------------------------
# decomposed collectives with autograd (gloo / CPU path)
# ------------------------------------------------------------------------------------------------
class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist

        ctx.group = group
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        world = dist.get_world_size(ctx.group) if dist.is_initialized() else 1
        if world == 1:
            return g, None
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        rows = g.size(0) // world
        r = dist.get_rank(ctx.group)
        return g[r * rows:(r + 1) * rows], None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, group):
        import torch.distributed as dist

        ctx.group = group
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world == 1:
            return y
        y = y.contiguous().clone()
        dist.all_reduce(y, group=group)
        rows = y.size(0) // world
        r = dist.get_rank(group)
        return y[r * rows:(r + 1) * rows].clone()

    @staticmethod
    def backward(ctx, g):
        return _GatherRows.apply(g, ctx.group), None


def _gather_rows(x, group):
    return _GatherRows.apply(x, group)


def _reduce_scatter_rows(y, group):
    return _ReduceScatterRows.apply(y, group)


class TPMLP(nn.Module):
    """SwiGLU feed-forward under TP + SP: gate/up column-parallel (interleaved per rank), down row-parallel."""

    def __init__(self, hidden: int, inter: int, grp, world: int, group=None):
        super().__init__()
        self.inter_local = inter // world
        self.gate_up = ColumnParallelLinear(hidden, 2 * inter, grp, world, group)     # this rank's [gate | up] halves
        self.down = RowParallelLinear(inter, hidden, grp, world, group)

    def forward(self, x_shard, resid=None):
        h = self.gate_up(x_shard)
        return self.down(block_ops.swiglu(h), resid)
