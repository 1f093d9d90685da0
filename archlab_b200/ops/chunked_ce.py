"""Full-vocabulary cross entropy with a TRAINABLE head, without ever holding more than one chunk of logits.

Forward: the summed loss over labelled tokens (-100: ignored), computed chunk by chunk from ``hidden`` and the head
weight; only ``hidden``, ``labels`` and ``weight`` are kept.  Backward: every chunk's logits are recomputed once, turned
into ``softmax - onehot`` in place, and used twice -- ``d hidden[chunk] = dlogits @ W`` and ``dW += dlogits^T @ hidden[chunk]``
(fp32 accumulation).  At a 129 k vocabulary this replaces a [tokens, vocab] fp32 activation by a [chunk, vocab] scratch,
at the price of one extra head GEMM.  On bf16 CUDA inputs the chunk products go through the framework's tensor-core
GEMM path (``F.linear`` dispatches there for converted linears); the function itself is device-agnostic.
(Reference: src/archlab/automodel/deepseek_v41_full_boundaries.py:48-117.)
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


class ChunkedHeadCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, labels, weight, chunk_tokens=1024):
        if type(chunk_tokens) is not int or chunk_tokens < 1:
            raise ValueError("chunk_tokens must be a positive integer")
        if hidden.shape[:-1] != labels.shape or hidden.shape[-1] != weight.shape[1]:
            raise ValueError("hidden / label / head shapes do not match")
        x, y = hidden.reshape(-1, hidden.shape[-1]), labels.reshape(-1)
        rows = torch.nonzero(y != -100, as_tuple=True)[0]
        loss = torch.zeros((), dtype=torch.float32, device=hidden.device)
        for ids in rows.split(chunk_tokens):
            loss += F.cross_entropy(F.linear(x[ids], weight).float(), y[ids], reduction="sum")
        ctx.save_for_backward(hidden, labels, weight)
        ctx.chunk = chunk_tokens
        return loss

    @staticmethod
    def backward(ctx, upstream):
        hidden, labels, weight = ctx.saved_tensors
        x, y = hidden.reshape(-1, hidden.shape[-1]), labels.reshape(-1)
        rows = torch.nonzero(y != -100, as_tuple=True)[0]
        need_x, _, need_w, _ = ctx.needs_input_grad
        dx = torch.zeros_like(x) if need_x else None
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device) if need_w else None
        scale = upstream.float()
        for ids in rows.split(ctx.chunk):
            xs = x[ids]
            d = torch.softmax(F.linear(xs, weight).float(), -1)
            d.scatter_add_(-1, y[ids, None], torch.full_like(d[:, :1], -1.0))
            d.mul_(scale)
            low = d.to(weight.dtype)
            if need_x:
                dx[ids] = (low @ weight).to(dx.dtype)
            if need_w:
                dw.addmm_(low.t().float() if weight.dtype == torch.float32 else low.t().to(torch.float32), xs.float())
        return (dx.view(hidden.shape) if need_x else None), None, (dw.to(weight.dtype) if need_w else None), None


def chunked_head_cross_entropy(hidden, labels, weight, *, chunk_tokens: int = 1024, reduction: str = "mean"):
    total = ChunkedHeadCrossEntropy.apply(hidden, labels, weight, chunk_tokens)
    if reduction == "sum":
        return total
    if reduction != "mean":
        raise ValueError("reduction is 'sum' or 'mean'")
    return total / (labels != -100).sum().clamp_min(1)
