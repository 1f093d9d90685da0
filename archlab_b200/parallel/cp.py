"""Context parallelism for causal attention: zig-zag sequence shards with gathered keys and values.

The sequence is cut into ``2 x CP`` equal chunks; rank ``r`` owns chunks ``r`` and ``2 CP - 1 - r`` so
that every rank does the same amount of causal work.  Keys and values are all-gathered over the
context group (their gradients are reduce-scattered back); each owned query chunk then attends to the
prefix of the gathered sequence it may see.  Positions (for RoPE) follow the owned chunks.

Plays the part of Megatron's ``--context-parallel-size`` in the reference's long-context launches
(``qwen38_flash_next_config.py:205-221``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


def zigzag_chunks(rank: int, world: int) -> tuple[int, int]:
    return rank, 2 * world - 1 - rank


def shard_sequence(x: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """The two zig-zag chunks of ``x`` along ``dim`` owned by ``rank``, concatenated."""
    if x.size(dim) % (2 * world):
        raise ValueError("sequence length must be a multiple of 2 x context-parallel size")
    parts = x.chunk(2 * world, dim)
    a, b = zigzag_chunks(rank, world)
    return torch.cat([parts[a], parts[b]], dim)


def shard_positions(T: int, rank: int, world: int, device=None) -> torch.Tensor:
    return shard_sequence(torch.arange(T, device=device)[None], rank, world)[0]


class _GatherSeq(torch.autograd.Function):
    """All-gather zig-zag shards into sequence order; backward reduce-scatters in the same layout."""

    @staticmethod
    def forward(ctx, x, world, group):
        ctx.world, ctx.group = world, group
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        L = x.size(1) // 2
        chunks = [None] * (2 * world)
        for r, p in enumerate(parts):
            a, b = zigzag_chunks(r, world)
            chunks[a], chunks[b] = p[:, :L], p[:, L:]
        return torch.cat(chunks, 1)

    @staticmethod
    def backward(ctx, g):
        world = ctx.world
        chunks = g.chunk(2 * world, 1)
        ins = [torch.cat([chunks[a], chunks[b]], 1).contiguous() for a, b in (zigzag_chunks(r, world) for r in range(world))]
        out = torch.empty_like(ins[0])
        if dist.get_backend(ctx.group) == "gloo":
            stacked = torch.stack(ins)
            dist.all_reduce(stacked, group=ctx.group)
            out = stacked[dist.get_rank(ctx.group)]
        else:
            dist.reduce_scatter(out, ins, group=ctx.group)
        return out, None, None


def gather_sequence(x: torch.Tensor, world: int, group=None) -> torch.Tensor:
    return x if world == 1 else _GatherSeq.apply(x, world, group)


def cp_causal_attention(q, k, v, *, rank: int, world: int, group=None, scale: float | None = None,
                        attend=None) -> torch.Tensor:
    """q [B, 2L, Hq, D], k/v [B, 2L, Hkv, D]: this rank's zig-zag shard.  Returns [B, 2L, Hq, D].

    ``attend(q_chunk, k_prefix, v_prefix, q_start)`` computes causal attention of a query chunk that
    starts at absolute position ``q_start`` against keys ``[0, q_start + L)``; the default is a masked
    softmax in PyTorch.
    """
    if world == 1:
        fn = attend or _prefix_attention
        return fn(q, k, v, 0, scale)
    L = q.size(1) // 2
    kf, vf = gather_sequence(k, world, group), gather_sequence(v, world, group)
    fn = attend or _prefix_attention
    outs = []
    for half, c in enumerate(zigzag_chunks(rank, world)):
        end = (c + 1) * L
        outs.append(fn(q[:, half * L:(half + 1) * L], kf[:, :end], vf[:, :end], c * L, scale))
    return torch.cat(outs, 1)


def _prefix_attention(q, k, v, q_start, scale=None):
    Tq, Tk = q.size(1), k.size(1)
    rep = q.size(2) // k.size(2)
    kk, vv = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
    qi = torch.arange(Tq, device=q.device)[:, None] + q_start
    mask = torch.arange(Tk, device=q.device)[None, :] <= qi
    o = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), attn_mask=mask, scale=scale)
    return o.transpose(1, 2)
