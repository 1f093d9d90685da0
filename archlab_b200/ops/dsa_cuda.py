"""Selected-key multi-query attention with a per-head sink on the tcgen05 flash kernels.

The lightning indexer picks, per query token, a set of visible keys shared by all heads.  Here the set
becomes one bit per (query, key) - ``[B, T, T/32]`` words, plus the key-major transpose for the
key-owned backward kernel - and the dense flash kernels skip the unselected entries in their softmax
stage.  For the configurations this framework trains (top-k at half the sequence or more) that is
cheaper than gathering 2048 rows per query, and it keeps the products on 128 x 128 tensor-core tiles.
Keys double as values (one shared latent head).  The sink adds ``exp(sink_h)`` to every row's
denominator; its gradient follows from the saved log-sum-exp and the row dot products dO . O.

Oracle: ``ops.dsa.sparse_attention`` / ``dense_sink_attention`` (the reference's
``query_chunked_sparse_attention``, src/archlab/automodel/deepseek_v41_torch.py:55-78).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import native, trunk

native.register_signature("nga_attn_fwd_set_extras", [C.c_void_p, C.c_void_p], None)
native.register_signature("nga_attn_bwd_set_extras", [C.c_void_p], None)
native.register_signature("nga_indexer_select", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                 C.c_int, C.c_float, C.c_void_p])
LOG2E = 1.4426950408889634


def kernel_supports(q: torch.Tensor, kv: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.size(-1) == 128 and q.size(1) % 128 == 0 and q.size(1) == kv.size(1)
            and native.available())


def _pack_bits(mask: torch.Tensor) -> torch.Tensor:
    """bool [..., T] -> int32 [..., T/32], bit i of word w = mask[..., 32 w + i]."""
    T = mask.size(-1)
    weights = (1 << torch.arange(8, device=mask.device)).to(torch.uint8)
    by = (mask.view(*mask.shape[:-1], T // 8, 8).to(torch.uint8) * weights).sum(-1, dtype=torch.uint8)     # byte j = bits 8j .. 8j+7
    return by.contiguous().view(torch.int32)                                                               # little-endian words


def selection_bits(indices: torch.Tensor, T: int):
    """indices [B, T, K] (negative = unused slot) -> (query-major bits, key-major bits), restricted to causal pairs."""
    B = indices.size(0)
    mask = torch.zeros(B, T, T + 1, dtype=torch.bool, device=indices.device)
    mask.scatter_(2, torch.where(indices < 0, T, indices).long(), True)
    mask = mask[..., :T]
    pos = torch.arange(T, device=indices.device)
    mask = mask & (pos[None, :] <= pos[:, None])
    return _pack_bits(mask), _pack_bits(mask.transpose(1, 2).contiguous())


class _SelectedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, sink, bits, bits_t):
        B, T, H, D = q.shape
        kv2 = kv.reshape(B * T, D)
        qkv = torch.cat([q.reshape(B * T, H * D), kv2, kv2], 1)
        sink32 = sink.detach().float().contiguous()
        lib = native.lib()
        lib.nga_attn_fwd_set_extras(None if bits is None else bits.data_ptr(), sink32.data_ptr())
        out, lse2 = trunk.attn_fwd(qkv, B, T, H, 1, D, -1)
        ctx.save_for_backward(qkv, out, lse2, sink32)
        ctx.bits_t, ctx.geom = bits_t, (B, T, H, D)
        return out.view(B, T, H, D)

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse2, sink32 = ctx.saved_tensors
        B, T, H, D = ctx.geom
        delta = torch.empty(B, H, T, dtype=torch.float32, device=qkv.device)
        native.lib().nga_attn_bwd_set_extras(None if ctx.bits_t is None else ctx.bits_t.data_ptr())
        dqkv = trunk.attn_bwd(qkv, out, dout.reshape(B * T, H * D).contiguous(), lse2, B, T, H, 1, D, -1, delta=delta)
        dq, dk, dv = dqkv.split([H * D, D, D], 1)
        p_sink = torch.exp2(sink32.view(1, H, 1) * LOG2E - lse2)             # probability each row gave the sink
        dsink = -(p_sink * delta).sum((0, 2))
        return dq.reshape(B, T, H, D), (dk + dv).reshape(B, T, D), dsink.to(sink32.dtype), None, None


def indexer_kernel_supports(q: torch.Tensor, k: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.size(2) == 4 and q.size(3) == 64 and q.size(1) % 32 == 0
            and q.size(1) <= 8192 and native.available())


def transpose_bits(bits: torch.Tensor, T: int) -> torch.Tensor:
    """[B, T, T/32] query-major selection words -> key-major words."""
    by = bits.contiguous().view(torch.uint8)                                   # [B, T, T/8]
    mask = ((by.unsqueeze(-1) >> torch.arange(8, device=bits.device, dtype=torch.uint8)) & 1).bool().view(bits.size(0), T, T)
    return _pack_bits(mask.transpose(1, 2).contiguous())


@torch.no_grad()
def indexer_select(q, k, w, top_k: int, scale: float | None = None):
    """q [B, S, 4, 64] bf16, k [B, S, 64] bf16, w [B, S, 4] -> (bits, key-major bits) of the causal top-k keys per
    query (threshold semantics: every key scoring at least the k-th largest score)."""
    B, S, H, D = q.shape
    bits = torch.empty(B, S, S // 32, dtype=torch.int32, device=q.device)
    rc = native.lib().nga_indexer_select(q.contiguous().data_ptr(), k.contiguous().data_ptr(), w.float().contiguous().data_ptr(),
                                         bits.data_ptr(), B, S, H, D, int(top_k), float(D ** -0.5 if scale is None else scale),
                                         native.stream_ptr())
    native.check(rc, "nga_indexer_select")
    return bits, transpose_bits(bits, S)


def selection_bits_from_scores(scores: torch.Tensor, kth: torch.Tensor):
    """scores [B, T, T] (-inf on non-causal pairs), kth [B, T, 1] the k-th largest score of every row (-inf when the
    row has fewer than k candidates): keys scoring at least the threshold are selected - no index scatter."""
    mask = (scores >= kth) & torch.isfinite(scores)
    return _pack_bits(mask), _pack_bits(mask.transpose(1, 2).contiguous())


def selected_sink_attention(q, kv, sink, indices=None, *, scores=None, kth=None, bits_pair=None):
    """q [B, T, H, 128], kv [B, T, 128] (key = value), sink [H]; the selection is given by ready ``bits_pair``
    (query-major, key-major), by ``indices`` [B, T, K], or by the indexer ``scores`` with their per-row threshold
    ``kth``; none of them: all causal keys."""
    bits = bits_t = None
    if bits_pair is not None:
        bits, bits_t = bits_pair
    elif scores is not None and kth is not None:
        bits, bits_t = selection_bits_from_scores(scores, kth)
    elif indices is not None:
        bits, bits_t = selection_bits(indices, q.size(1))
    return _SelectedAttention.apply(q, kv.to(q.dtype), sink, bits, bits_t)
