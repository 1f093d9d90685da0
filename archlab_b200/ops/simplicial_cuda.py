"""CUDA binding of the 2-simplicial attention kernels (``csrc/simplicial_fwd.cu`` /
``simplicial_bwd.cu``) as a ``torch.autograd.Function``."""
from __future__ import annotations

import ctypes as C

import torch

from . import native

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
native.register_signature("nga_simplicial_fwd", [_vp] * 7 + [_ll] * 6 + [_i] * 7 + [_f, _vp, _vp])
native.register_signature("nga_simplicial_bwd", [_vp] * 18 + [_ll] * 12 + [_i] * 7 + [_f, _vp, _vp])


def kernel_supports(q, k1, v1, w1: int, w2: int) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and v1.shape[-1] == 128
            and w1 in (8, 16, 32) and w2 >= w1 and native.available())


def _rows(t: torch.Tensor):
    """[B, N, H, D] tensor with contiguous (H, D) -> (data_ptr, row stride in elements)."""
    B, N, H, D = t.shape
    if t.stride(3) != 1 or t.stride(2) != D or t.stride(0) != N * t.stride(1):
        t = t.contiguous()
    return t, t.stride(1)


def simplicial_fwd(q, k1, k2, v1, v2, w1, w2, scale):
    B, N, Hq, D = q.shape
    Hkv = k1.shape[2]
    (q, ldq), (k1, ldk1), (k2, ldk2), (v1, ldv1), (v2, ldv2) = (_rows(t) for t in (q, k1, k2, v1, v2))
    out = torch.empty(B, N, Hq, D, dtype=torch.bfloat16, device=q.device)
    lse2 = torch.empty(B, Hq, N, dtype=torch.float32, device=q.device)
    rc = native.lib().nga_simplicial_fwd(q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(),
                                         out.data_ptr(), lse2.data_ptr(), ldq, ldk1, ldk2, ldv1, ldv2, Hq * D, B, N,
                                         Hq, Hkv, D, w1, w2, scale, native.status_word(q.device).data_ptr(),
                                         native.stream_ptr())
    native.check(rc, "nga_simplicial_fwd")
    return out, lse2


class SimplicialFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k1, k2, v1, v2, w1, w2, scale):
        out, lse2 = simplicial_fwd(q, k1, k2, v1, v2, w1, w2, scale)
        ctx.save_for_backward(q, k1, k2, v1, v2, out, lse2)
        ctx.cfg = (w1, w2, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k1, k2, v1, v2, out, lse2 = ctx.saved_tensors
        w1, w2, scale = ctx.cfg
        if hasattr(native.lib(), "nga_simplicial_bwd"):
            from .simplicial_bwd import simplicial_bwd

            dq, dk1, dk2, dv1, dv2 = simplicial_bwd(q, k1, k2, v1, v2, out, dout.contiguous(), lse2, w1, w2, scale)
            return dq, dk1, dk2, dv1, dv2, None, None, None
        # recompute through the differentiable PyTorch statement (fp32)
        from .simplicial import simplicial_attention_reference

        with torch.enable_grad():
            ins = [t.detach().float().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
            ref = simplicial_attention_reference(*ins, w1, w2, scale=scale)
            grads = torch.autograd.grad(ref, ins, dout.float())
        return (*[g.to(torch.bfloat16) for g in grads], None, None, None)
