"""Causal (optionally windowed) grouped-query attention as an autograd op over the tcgen05 kernels.

``causal_attention(q, k, v, window=-1)`` takes q [B, T, Hq, D], k/v [B, T, Hkv, D].  On CUDA with
bf16 inputs and head_dim 128 the forward and backward run the hand-written flash kernels (the
operands are packed once into the [B*T, (Hq + 2 Hkv) * D] layout those kernels read; the packed
gradient is split back).  Elsewhere the masked-softmax definition in PyTorch runs (the oracle).
Stands where the reference calls FlashAttention through ``TorchAttentionOps``
(src/archlab/architectures/base.py:26-87).
"""
from __future__ import annotations

import torch

from . import trunk


def kernel_supports(q: torch.Tensor, k: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.size(-1) == 128 and q.size(1) % 128 == 0
            and q.size(2) % k.size(2) == 0)


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, window):
        B, T, Hq, D = q.shape
        Hkv = k.size(2)
        qkv = torch.cat([q.reshape(B * T, Hq * D), k.reshape(B * T, Hkv * D), v.reshape(B * T, Hkv * D)], 1)
        out, lse2 = trunk.attn_fwd(qkv, B, T, Hq, Hkv, D, window)
        ctx.save_for_backward(qkv, out, lse2)
        ctx.geom = (B, T, Hq, Hkv, D, window)
        return out.view(B, T, Hq, D)

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse2 = ctx.saved_tensors
        B, T, Hq, Hkv, D, window = ctx.geom
        dqkv = trunk.attn_bwd(qkv, out, dout.reshape(B * T, Hq * D).contiguous(), lse2, B, T, Hq, Hkv, D, window)
        dq, dk, dv = dqkv.split([Hq * D, Hkv * D, Hkv * D], 1)
        return dq.reshape(B, T, Hq, D), dk.reshape(B, T, Hkv, D), dv.reshape(B, T, Hkv, D), None


def causal_attention(q, k, v, window: int = -1) -> torch.Tensor:
    if kernel_supports(q, k):
        return _FlashFn.apply(q, k.to(q.dtype), v.to(q.dtype), int(window))
    return trunk.attention_reference(q, k, v, window).to(q.dtype)
