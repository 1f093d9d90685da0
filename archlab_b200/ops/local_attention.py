"""Causal sliding-window GQA attention (the matched ``local`` control of the simplicial branches).

``reference_local_attention`` is the explicit fp32 softmax statement
(src/archlab/architectures/local_attention.py:27-40); ``local_attention`` dispatches to the sm_100a
attention kernels for bf16 / head_dim 128 CUDA inputs and to the statement otherwise.  ``window``
counts the keys a query sees, itself included.
"""
from __future__ import annotations

import math

import torch


def _check(q, k, v, window):
    if q.ndim != 4 or k.ndim != 4 or k.shape != v.shape or k.shape[:2] != q.shape[:2] or window < 1:
        raise ValueError("expected [B, T, H, D] tensors and a positive window")
    if k.shape[-1] != q.shape[-1] or k.shape[2] < 1 or q.shape[2] % k.shape[2]:
        raise ValueError("incompatible grouped-query attention shapes")


def reference_local_attention(q, k, v, window: int):
    _check(q, k, v, window)
    rep = q.shape[2] // k.shape[2]
    qf = q.float().transpose(1, 2)
    kf = k.float().repeat_interleave(rep, 2).transpose(1, 2)
    vf = v.float().repeat_interleave(rep, 2).transpose(1, 2)
    T = q.shape[1]
    i = torch.arange(T, device=q.device)
    mask = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < window)
    s = (qf @ kf.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    p = s.masked_fill(~mask, float("-inf")).softmax(-1)
    return (p @ vf).transpose(1, 2).to(q.dtype)


class _LocalAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, window):
        from . import trunk

        B, T, Hq, D = q.shape
        Hkv = k.shape[2]
        qkv = torch.cat([q.reshape(B * T, Hq * D), k.reshape(B * T, Hkv * D), v.reshape(B * T, Hkv * D)], 1).contiguous()
        out, lse2 = trunk.attn_fwd(qkv, B, T, Hq, Hkv, D, window - 1)
        ctx.save_for_backward(qkv, out, lse2)
        ctx.geom = (B, T, Hq, Hkv, D, window - 1)
        return out.view(B, T, Hq, D)

    @staticmethod
    def backward(ctx, dout):
        from . import trunk

        qkv, out, lse2 = ctx.saved_tensors
        B, T, Hq, Hkv, D, w = ctx.geom
        d = trunk.attn_bwd(qkv, out, dout.reshape(B * T, Hq * D).contiguous(), lse2, B, T, Hq, Hkv, D, w)
        dq, dk, dv = d.split((Hq * D, Hkv * D, Hkv * D), 1)
        return dq.reshape(B, T, Hq, D), dk.reshape(B, T, Hkv, D), dv.reshape(B, T, Hkv, D), None


def local_attention(q, k, v, window: int):
    _check(q, k, v, window)
    from . import native

    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and native.available():
        return _LocalAttentionFn.apply(q, k, v, window)
    return reference_local_attention(q, k, v, window)
