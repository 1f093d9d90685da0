"""Thin Python launchers for the memory-bound trunk kernels (``csrc/elementwise.cu``) and the
attention kernels (``csrc/attention_fwd.cu`` / ``attention_bwd.cu``), each paired with a plain
fp32 PyTorch statement of the same arithmetic that serves as the oracle in the GPU tests and as
the CPU execution path.
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.nn.functional as F

from . import native

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float

native.register_signature("nga_mix_norm_fwd", [_vp, _vp, _vp, _vp, _f, _f, _vp, _vp, _ll, _i, _vp])
native.register_signature("nga_norm_bwd", [_vp, _vp, _vp, _vp, _i, _vp, _vp, _f, _f, _vp, _vp, _vp, _i,
                                           _vp, _vp, _ll, _i, _vp])
native.register_signature("nga_embed_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _vp])
native.register_signature("nga_embed_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i,
                                            _i, _vp])
native.register_signature("nga_qkv_post_fwd", [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp,
                                               _ll, _i, _i, _i, _i, _vp])
native.register_signature("nga_qkv_post_bwd", [_vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp,
                                               _ll, _i, _i, _i, _i, _vp])
native.register_signature("nga_gate_bwd", [_vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _vp])
native.register_signature("nga_softcap_ce", [_vp, _vp, _vp, _f, _f, _ll, _ll, _i, _vp])
native.register_signature("nga_attn_fwd", [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _vp])
native.register_signature("nga_attn_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                           _f, _vp, _vp])


native.register_signature("nga_axpby_bf16", [_vp, _vp, _f, _f, _ll, _vp])
native.register_signature("nga_cast_f32_bf16", [_vp, _vp, _ll, _vp])


def _p(t):
    return None if t is None else t.data_ptr()


def _s():
    return native.stream_ptr()


# ------------------------------------------------------------------------------------------------
# mix + norm
# ------------------------------------------------------------------------------------------------
def rms(x: torch.Tensor) -> torch.Tensor:
    return F.rms_norm(x.float(), (x.size(-1),)).to(x.dtype)


def mix_norm_fwd(x, x0=None, a=None, b=None, a_scale=1.0, b_scale=1.0):
    """x1 = a_scale*a*x + b_scale*b*x0 (skipped when x0 is None); returns (x1, rmsnorm(x1))."""
    if x.device.type != "cuda":
        if x0 is None:
            return x, rms(x)
        av = a_scale * (float(a) if a is not None else 1.0)
        bv = b_scale * (float(b) if b is not None else 0.0)
        x1 = (av * x.float() + bv * x0.float()).to(x.dtype)
        return x1, rms(x1)
    rows, Cc = x.numel() // x.size(-1), x.size(-1)
    x1 = torch.empty_like(x) if x0 is not None else x
    n = torch.empty_like(x)
    rc = native.lib().nga_mix_norm_fwd(_p(x), _p(x0), _p(a), _p(b), a_scale, b_scale, _p(x1), _p(n),
                                       rows, Cc, _s())
    native.check(rc, "nga_mix_norm_fwd")
    return x1, n


def norm_bwd(x, dn, dres=None):
    """Gradient of n = rmsnorm(x) plus an optional residual gradient."""
    if x.device.type != "cuda":
        xf = x.float().detach().requires_grad_(True)
        y = F.rms_norm(xf, (x.size(-1),))
        (g,) = torch.autograd.grad(y, xf, dn.float())
        if dres is not None:
            g = g + dres.float()
        return g.to(x.dtype)
    rows, Cc = x.numel() // x.size(-1), x.size(-1)
    dx = torch.empty_like(x)
    rc = native.lib().nga_norm_bwd(_p(x), _p(dn), _p(dres), _p(dx), 0, None, None, 1.0, 1.0, None, None,
                                   None, 0, None, None, rows, Cc, _s())
    native.check(rc, "nga_norm_bwd")
    return dx


def norm_bwd_mix(x1, dn, dres, a, b, xprev, x0, dx0, dx0_init, da, db, a_scale=1.0, b_scale=1.0):
    """Backward of ``x1 = a*xprev + b*x0; n = rmsnorm(x1)`` given dn and the residual gradient
    dres.  Returns dxprev; accumulates b*g into dx0 (bf16) and <g,xprev>, <g,x0> into da, db."""
    if x1.device.type != "cuda":
        g = norm_bwd(x1, dn, dres).float()
        av = a_scale * float(a)
        bv = b_scale * float(b)
        if dx0_init:
            dx0.copy_((bv * g).to(dx0.dtype))
        else:
            dx0.copy_((dx0.float() + bv * g).to(dx0.dtype))
        if da is not None:
            da.add_((g * xprev.float()).sum())
        if db is not None:
            db.add_((g * x0.float()).sum())
        return (av * g).to(x1.dtype)
    rows, Cc = x1.numel() // x1.size(-1), x1.size(-1)
    dx = torch.empty_like(x1)
    rc = native.lib().nga_norm_bwd(_p(x1), _p(dn), _p(dres), _p(dx), 1, _p(a), _p(b), a_scale, b_scale,
                                   _p(xprev), _p(x0), _p(dx0), int(dx0_init), _p(da), _p(db), rows, Cc,
                                   _s())
    native.check(rc, "nga_norm_bwd(mix)")
    return dx


# ------------------------------------------------------------------------------------------------
# embedding + norm + smear
# ------------------------------------------------------------------------------------------------
def embed_fwd(idx, wte, gate_w, lam, T):
    rows, Cc = idx.numel(), wte.size(1)
    x0 = torch.empty(rows, Cc, dtype=torch.bfloat16, device=idx.device)
    gate_pre = torch.empty(rows, dtype=torch.float32, device=idx.device)
    rc = native.lib().nga_embed_fwd(_p(idx), _p(wte), _p(gate_w), _p(lam), _p(x0), _p(gate_pre), rows, T,
                                    Cc, gate_w.numel(), _s())
    native.check(rc, "nga_embed_fwd")
    return x0, gate_pre


def embed_bwd(idx, wte, gate_w, lam, gate_pre, g, dwte, dgate_w, dlam, T):
    rows, Cc = idx.numel(), wte.size(1)
    rc = native.lib().nga_embed_bwd(_p(idx), _p(wte), _p(gate_w), _p(lam), _p(gate_pre), _p(g), _p(dwte),
                                    _p(dgate_w), _p(dlam), rows, T, Cc, gate_w.numel(), _s())
    native.check(rc, "nga_embed_bwd")


def embed_reference(idx, wte, gate_w, lam):
    """idx [B, T]; returns x0 [B, T, C] (autograd-capable fp32 math, bf16 rounding where the
    reference model rounds)."""
    e = F.rms_norm(wte[idx].float(), (wte.size(1),)).to(torch.bfloat16).float()
    G = gate_w.numel()
    gate = lam.float() * torch.sigmoid(e[:, 1:, :G] @ gate_w.float().view(-1, 1))
    return torch.cat([e[:, :1], e[:, 1:] + gate * e[:, :-1]], dim=1)


# ------------------------------------------------------------------------------------------------
# qkv post-processing
# ------------------------------------------------------------------------------------------------
def qkv_post_fwd(qkv, cosT, sinT, gain, idx, ve_table, gate_w, n, T, Hq, Hkv, D):
    rows = qkv.size(0)
    rstd = torch.empty(rows, Hq + Hkv, dtype=torch.float32, device=qkv.device)
    gate_pre = None
    GC = 0
    if ve_table is not None:
        gate_pre = torch.empty(rows, Hkv, dtype=torch.float32, device=qkv.device)
        GC = gate_w.size(1)
    rc = native.lib().nga_qkv_post_fwd(_p(qkv), _p(cosT), _p(sinT), gain, _p(idx), _p(ve_table),
                                       _p(gate_w), _p(n), GC, n.size(1), _p(rstd), _p(gate_pre), rows, T,
                                       Hq, Hkv, D, _s())
    native.check(rc, "nga_qkv_post_fwd")
    return rstd, gate_pre


def qkv_post_bwd(dqkv, qkv, cosT, sinT, gain, idx, ve_table, rstd, gate_pre, dve_table, T, Hq, Hkv, D):
    rows = qkv.size(0)
    dgp = None
    if ve_table is not None:
        dgp = torch.empty(rows, Hkv, dtype=torch.float32, device=qkv.device)
    rc = native.lib().nga_qkv_post_bwd(_p(dqkv), _p(qkv), _p(cosT), _p(sinT), gain, _p(idx), _p(ve_table),
                                       _p(rstd), _p(gate_pre), _p(dgp), _p(dve_table), rows, T, Hq, Hkv,
                                       D, _s())
    native.check(rc, "nga_qkv_post_bwd")
    return dgp


def gate_bwd(dn, n, dgp, gate_w, dgate_w):
    rows, Cc = n.size(0), n.size(1)
    H, GC = gate_w.shape
    rc = native.lib().nga_gate_bwd(_p(dn), _p(n), _p(dgp), _p(gate_w), _p(dgate_w), rows, Cc, GC, H, _s())
    native.check(rc, "nga_gate_bwd")


# ------------------------------------------------------------------------------------------------
# soft-capped cross entropy (forward + gradient in place)
# ------------------------------------------------------------------------------------------------
def softcap_ce_(logits, targets, gscale, cap=15.0):
    """logits [n, V] bf16 is overwritten by d(loss)/d(logits) * gscale; returns per-row losses."""
    n, V = logits.shape
    loss_rows = torch.empty(n, dtype=torch.float32, device=logits.device)
    rc = native.lib().nga_softcap_ce(_p(logits), _p(targets), _p(loss_rows), cap, gscale, n,
                                     logits.stride(0), V, _s())
    native.check(rc, "nga_softcap_ce")
    return loss_rows


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
def attn_fwd(qkv, B, T, Hq, Hkv, D, window):
    out = torch.empty(B * T, Hq * D, dtype=torch.bfloat16, device=qkv.device)
    lse2 = torch.empty(B, Hq, T, dtype=torch.float32, device=qkv.device)
    rc = native.lib().nga_attn_fwd(_p(qkv), _p(out), _p(lse2), B, T, Hq, Hkv, D, window,
                                   1.0 / math.sqrt(D), native.status_word(qkv.device).data_ptr(), _s())
    native.check(rc, "nga_attn_fwd")
    return out, lse2


def attn_bwd(qkv, out, dout, lse2, B, T, Hq, Hkv, D, window, dq_acc=None, delta=None):
    dqkv = torch.empty_like(qkv)
    if dq_acc is None:
        dq_acc = torch.empty(B * T, Hq * D, dtype=torch.float32, device=qkv.device)
    if delta is None:
        delta = torch.empty(B, Hq, T, dtype=torch.float32, device=qkv.device)
    rc = native.lib().nga_attn_bwd(_p(qkv), _p(out), _p(dout), _p(lse2), _p(dqkv), _p(dq_acc), _p(delta),
                                   B, T, Hq, Hkv, D, window, 1.0 / math.sqrt(D),
                                   native.status_word(qkv.device).data_ptr(), _s())
    native.check(rc, "nga_attn_bwd")
    return dqkv


def attention_reference(q, k, v, window):
    """q [B,T,Hq,D], k/v [B,T,Hkv,D] -> [B,T,Hq,D]; the masked-softmax definition in fp32."""
    B, T, Hq, D = q.shape
    Hkv = k.size(2)
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    if Hkv != Hq:
        kf = kf.repeat_interleave(Hq // Hkv, dim=1)
        vf = vf.repeat_interleave(Hq // Hkv, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    i = torch.arange(T, device=q.device).view(T, 1)
    j = torch.arange(T, device=q.device).view(1, T)
    mask = j <= i
    if window >= 0:
        mask = mask & ((i - j) <= window)
    s = s.masked_fill(~mask, float("-inf"))
    return (torch.softmax(s, dim=-1) @ vf).transpose(1, 2)


def axpby_(y, x, a=1.0, b=1.0):
    """y = a * x + b * y in place (bf16)."""
    rc = native.lib().nga_axpby_bf16(_p(x), _p(y), a, b, y.numel(), _s())
    native.check(rc, "nga_axpby_bf16")
    return y


def cast_to_bf16_(dst, src):
    """dst (bf16) = src (fp32), same number of elements (a multiple of 4)."""
    rc = native.lib().nga_cast_f32_bf16(_p(src), _p(dst), src.numel(), _s())
    native.check(rc, "nga_cast_f32_bf16")
    return dst
