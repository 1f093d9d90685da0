"""Autograd forms of the per-block operators on the sm_100a kernels: RMSNorm (with gain), rotary
embedding, SwiGLU on a packed [gate | up] tensor, and cross-entropy that leaves the logit gradient
in place of the logits.  Each is one kernel forward and one backward; off the GPU (or for shapes the
kernels do not take) the PyTorch statements in ``models.blocks`` run instead.

They stand where the reference composes ``apply_qk_features`` / ``RMSNorm`` / ``MLP`` /
``language_model_loss`` from eager PyTorch ops under ``torch.compile``
(src/archlab/architectures/base.py:150-181,231-265,362-366).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import native

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
native.register_signature("nga_rmsnorm", [_vp, _vp, _vp, _ll, _i, _i, _f, _i, _vp])
native.register_signature("nga_rmsnorm_bwd", [_vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _f, _i, _vp])
native.register_signature("nga_rope", [_vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _vp])
native.register_signature("nga_swiglu_clamped", [_vp, _vp, _vp, _ll, _i, _f, _vp])
native.register_signature("nga_swiglu_bwd", [_vp, _vp, _vp, _ll, _i, _f, _vp])
native.register_signature("nga_ce_inplace", [_vp, _vp, _vp, _f, _ll, _ll, _i, _ll, _vp])


def _p(t):
    return None if t is None else t.data_ptr()


def usable(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and native.available()


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, zero_centered, groups):
        x = x.contiguous()
        width = x.size(-1) // groups
        rows = x.numel() // x.size(-1)
        wf = None if weight is None else weight.detach().float().contiguous()
        y = torch.empty_like(x)
        native.check(native.lib().nga_rmsnorm(_p(x), _p(wf), _p(y), rows, groups, width, eps, int(zero_centered),
                                              native.stream_ptr()), "nga_rmsnorm")
        ctx.save_for_backward(x, wf)
        ctx.meta = (rows, groups, width, eps, zero_centered, None if weight is None else weight.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wf = ctx.saved_tensors
        rows, groups, width, eps, zc, wdtype = ctx.meta
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros(groups * width, dtype=torch.float32, device=x.device) if wf is not None else None
        native.check(native.lib().nga_rmsnorm_bwd(_p(x), _p(wf), _p(dy), _p(dx), _p(dw), rows, groups, width, eps, int(zc),
                                                  native.stream_ptr()), "nga_rmsnorm_bwd")
        return dx, (None if dw is None else dw.to(wdtype)), None, None, None


def rms_norm(x, weight=None, *, eps: float = 1e-6, zero_centered: bool = False, groups: int = 1):
    """x [..., groups * width] -> same shape; weight [groups * width] or None."""
    return _RMSNorm.apply(x, weight, float(eps), bool(zero_centered), int(groups))


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, rot, interleaved):
        B, T, H, D = x.shape
        cos, sin = cos.float().contiguous(), sin.float().contiguous()
        y = x.contiguous().clone()
        native.check(native.lib().nga_rope(_p(y), _p(cos), _p(sin), B * T, T, H, D, rot, int(interleaved), native.stream_ptr()),
                     "nga_rope")
        ctx.save_for_backward(cos, sin)
        ctx.meta = (B, T, H, D, rot, interleaved)
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        B, T, H, D, rot, interleaved = ctx.meta
        dx = dy.contiguous().clone()
        native.check(native.lib().nga_rope(_p(dx), _p(cos), _p((-sin).contiguous()), B * T, T, H, D, rot, int(interleaved),
                                           native.stream_ptr()), "nga_rope")        # the inverse rotation
        return dx, None, None, None, None


def rope(x, cos, sin, *, rot_dim=None, interleaved: bool = False):
    """x [B, T, H, D] bf16, tables [T, rot/2] (row t of the tables belongs to sequence position t)."""
    return _Rope.apply(x, cos, sin, x.size(-1) if rot_dim is None else int(rot_dim), bool(interleaved))


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, limit):
        h = h.contiguous()
        rows, inter = h.numel() // h.size(-1), h.size(-1) // 2
        out = torch.empty(*h.shape[:-1], inter, dtype=h.dtype, device=h.device)
        native.check(native.lib().nga_swiglu_clamped(_p(h), None, _p(out), rows, inter, limit, native.stream_ptr()),
                     "nga_swiglu_clamped")
        ctx.save_for_backward(h)
        ctx.meta = (rows, inter, limit)
        return out

    @staticmethod
    def backward(ctx, dout):
        (h,) = ctx.saved_tensors
        rows, inter, limit = ctx.meta
        dh = torch.empty_like(h)
        if rows == 0:                      # a rank without expert rows still runs the backward of its (empty) branch
            return dh, None
        native.check(native.lib().nga_swiglu_bwd(_p(h), _p(dout.contiguous()), _p(dh), rows, inter, limit, native.stream_ptr()),
                     "nga_swiglu_bwd")
        return dh, None


def swiglu(h, limit: float | None = None):
    """h [..., 2 * inter] packed [gate | up] -> silu(gate) * up (clamped when ``limit`` is given)."""
    if usable(h) and (h.size(-1) // 2) % 8 == 0:
        return _SwiGLU.apply(h, 0.0 if limit is None else float(limit))
    g, u = h.float().chunk(2, -1)
    if limit is not None:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return (torch.nn.functional.silu(g) * u).to(h.dtype)


class _CrossEntropySum(torch.autograd.Function):
    """Sum of the token losses; the bf16 logits buffer is overwritten with d(loss_sum)/d(logits)."""

    @staticmethod
    def forward(ctx, logits, targets, ignore_index):
        rows, V = logits.shape
        loss_rows = torch.empty(rows, dtype=torch.float32, device=logits.device)
        native.check(native.lib().nga_ce_inplace(_p(logits), _p(targets.contiguous()), _p(loss_rows), 1.0, rows,
                                                 logits.stride(0), V, ignore_index, native.stream_ptr()), "nga_ce_inplace")
        ctx.save_for_backward(logits)
        return loss_rows.sum()

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return grad.mul_(g.to(grad.dtype)), None, None


def cross_entropy_sum(logits, targets, ignore_index: int = -1):
    """logits [rows, V] (bf16 CUDA: consumed - do not reuse them afterwards), targets [rows] int64."""
    if usable(logits) and logits.dim() == 2 and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
        return _CrossEntropySum.apply(logits, targets.long(), int(ignore_index))
    return torch.nn.functional.cross_entropy(logits.float(), targets, ignore_index=ignore_index, reduction="sum")
