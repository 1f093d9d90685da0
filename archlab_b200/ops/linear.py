"""``y = x W^T`` as an autograd function on the tcgen05 GEMM: forward NT, input gradient NN (the
weight is read as the MN-major operand, no transposed copy), weight gradient TN.  Falls back to
``F.linear`` off the GPU or for non-bf16 inputs."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import gemm as G
from . import native


class _LinearBf16(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.size(-1))
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.shape = x.shape
        return G.gemm(x2, w).view(*x.shape[:-1], w.size(0))

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.size(-1))
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = G.gemm(g2, w, b_mn=True).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            gw = G.gemm(g2, x2, a_mn=True, b_mn=True)
        return gx, gw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    ok = (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and native.available()
          and x.size(-1) % 8 == 0 and w.size(0) % 8 == 0 and x.numel() > 0)
    if not ok:
        return F.linear(x, w.to(x.dtype))
    return _LinearBf16.apply(x, w if w.is_contiguous() else w.contiguous())
