"""Bias-free linear layers on the tcgen05 GEMM kernels for models written with ``nn.Linear``.

``y = x W^T`` (NT), ``dx = dy W`` (NN, W read MN-major in place) and ``dW = dy^T x`` (TN, both operands MN-major)
are the three orientations of ``ops.gemm.gemm``; no transposed copy is made.  ``convert_linears`` swaps the
eligible layers of a module tree in place (same parameter objects, so optimizers and checkpoints are unaffected).
On CPU the same calls run the fp32 PyTorch statement of the kernel, which is what the CPU tests compare against.
The fully-sharded form of the same layer is ``parallel.fsdp.FsdpLinear``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import gemm as G


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.size(-1))
        if x.is_cuda:
            x2, wc = x2.to(torch.bfloat16).contiguous(), w.to(torch.bfloat16)
        else:
            wc = w.to(x2.dtype)
        ctx.save_for_backward(x2, wc)
        ctx.lead, ctx.dtypes = x.shape[:-1], (x.dtype, w.dtype)
        y = G.gemm(x2, wc, out_dtype=x2.dtype)
        return y.reshape(*x.shape[:-1], w.size(0)).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x2, wc = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1)).to(x2.dtype).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(dy2, wc, b_mn=True, out_dtype=x2.dtype).reshape(*ctx.lead, wc.size(1)).to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            dw = G.gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=x2.dtype).to(ctx.dtypes[1])
        return dx, dw


def native_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return _LinearFn.apply(x, weight)


class NativeLinear(nn.Linear):
    """Drop-in ``nn.Linear(bias=False)`` whose three GEMMs run on the hand-written kernels."""

    def __init__(self, in_features: int, out_features: int, device=None, dtype=None):
        super().__init__(in_features, out_features, bias=False, device=device, dtype=dtype)

    def forward(self, x):
        return native_linear(x, self.weight)


def eligible(layer: nn.Module, min_features: int = 128) -> bool:
    """Plain bias-free linears (other subclasses keep their own forward) with sides that are multiples of 8 elements (16-byte
    rows for the tensor maps) and at least ``min_features`` wide."""
    from ..models.nanochat import CastLinear               # fp32 master weight, matmul in the activation dtype: same contract

    return (type(layer) in (nn.Linear, CastLinear) and layer.bias is None and layer.in_features % 8 == 0 and layer.out_features % 8 == 0
            and min(layer.in_features, layer.out_features) >= min_features)


def convert_linears(module: nn.Module, *, min_features: int = 128) -> list[str]:
    """Re-classes every eligible ``nn.Linear`` of ``module`` as ``NativeLinear`` in place; returns their names."""
    changed = []
    for name, layer in module.named_modules():
        if eligible(layer, min_features):
            layer.__class__ = NativeLinear
            changed.append(name)
    return changed
