"""Tensor-scaled FP8 linear layers on the tcgen05 ``kind::f8f6f4`` pair-CTA GEMM.

Forward: input and weight are scaled to the e4m3 range by one amax-derived factor each and multiplied
on the 8-bit tensor-core path (twice the bf16 rate); the product of the two inverse scales is the GEMM's
``alpha``.  Backward: the output gradient goes to e5m2 (range over precision); ``dX = dY W`` and
``dW = dY^T X`` reuse the saved 8-bit operands through transposed 8-bit copies, because the 8-bit
tensor-core path takes K-major operands only.  This is the arithmetic of the reference's
``Float8Linear`` (src/archlab/speedrun/fp8.py:88-235, which calls ``torch._scaled_mm``); here the
GEMM is the framework's own kernel.  Off the GPU the same quantise / de-quantise arithmetic runs in fp32.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn as nn

from . import native

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
native.register_signature("nga_gemm2_fp8", [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _i, _i, _i, _i, _f, _f, _vp, _vp])
E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


def quantize_tensorwise(x: torch.Tensor, dtype=E4M3):
    """-> (x in ``dtype``, inverse scale as an fp32 scalar tensor): x ~= x_q * inv_scale."""
    fmax = torch.finfo(dtype).max
    amax = x.detach().abs().amax().float().clamp_min(1e-12)
    scale = fmax / amax
    q = (x.float() * scale).clamp(-fmax, fmax).to(dtype)
    return q, scale.reciprocal()


def fp8_gemm(a_q: torch.Tensor, b_q: torch.Tensor, alpha: float, out_dtype=torch.bfloat16) -> torch.Tensor:
    """a_q [M, K], b_q [N, K] (8-bit floats, row-major) -> alpha * a b^T."""
    M, K = a_q.shape
    N = b_q.size(0)
    usable = a_q.is_cuda and K % 16 == 0 and native.available() and a_q.is_contiguous() and b_q.is_contiguous()
    if not usable:
        return (alpha * (a_q.float() @ b_q.float().t())).to(out_dtype)
    out = torch.empty(M, N, dtype=out_dtype, device=a_q.device)
    rc = native.lib().nga_gemm2_fp8(a_q.data_ptr(), b_q.data_ptr(), out.data_ptr(), None, M, N, K, a_q.stride(0), b_q.stride(0),
                                    out.stride(0), 0, int(a_q.dtype == E5M2), int(b_q.dtype == E5M2), 0, int(out_dtype == torch.float32),
                                    0, float(alpha), 0.0, native.status_word(a_q.device).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_gemm2_fp8")
    return out


class _Fp8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w):
        xq, xi = quantize_tensorwise(x2, E4M3)
        wq, wi = quantize_tensorwise(w, E4M3)
        ctx.save_for_backward(xq, xi, wq, wi)
        ctx.dtypes = (x2.dtype, w.dtype)
        return fp8_gemm(xq, wq, float(xi * wi), x2.dtype if x2.dtype != torch.float32 else torch.float32)

    @staticmethod
    def backward(ctx, g):
        xq, xi, wq, wi = ctx.saved_tensors
        xdt, wdt = ctx.dtypes
        gq, gi = quantize_tensorwise(g.contiguous(), E5M2)
        # dX [M, K] = dY [M, N] W [N, K]: the B operand must be [K, N] row-major
        dx = fp8_gemm(gq, wq.t().contiguous(), float(gi * wi), xdt if xdt != torch.float32 else torch.float32)
        # dW [N, K] = dY^T [N, M] X [M, K]: A = dY^T row-major, B = X^T row-major
        dw = fp8_gemm(gq.t().contiguous(), xq.t().contiguous(), float(gi * xi), torch.float32)
        return dx, dw.to(wdt)


def fp8_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    shape = x.shape
    y = _Fp8Linear.apply(x.reshape(-1, shape[-1]), weight)
    return y.view(*shape[:-1], weight.size(0))


class Float8Linear(nn.Linear):
    """Drop-in ``nn.Linear`` (no bias) whose three GEMMs run in FP8; parameters stay in their own dtype."""

    def forward(self, x):
        if self.bias is not None:
            raise ValueError("Float8Linear has no bias")
        return fp8_linear(x, self.weight.to(x.dtype) if x.dtype != torch.float32 else self.weight)


def convert_linears(module: nn.Module, *, min_features: int = 128, skip: tuple[str, ...] = ("lm_head",)) -> int:
    """Swap eligible ``nn.Linear`` children for ``Float8Linear`` in place (dims multiples of 16, no bias)."""
    n = 0
    for name, child in list(module.named_children()):
        if (type(child) is nn.Linear and child.bias is None and name not in skip and child.in_features % 16 == 0
                and child.out_features % 16 == 0 and min(child.in_features, child.out_features) >= min_features):
            new = Float8Linear(child.in_features, child.out_features, bias=False, device=child.weight.device, dtype=child.weight.dtype)
            new.weight = child.weight
            setattr(module, name, new)
            n += 1
        else:
            n += convert_linears(child, min_features=min_features, skip=skip)
    return n
