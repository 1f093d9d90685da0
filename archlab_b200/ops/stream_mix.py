"""Per-token mixing of residual streams on the sm_100a kernels, with autograd.

``token_mix(W, a, b=None)``: ``out[..., o, :] = sum_j W[..., o, j] * rows[..., j, :]`` where ``rows`` are the
``na`` rows of ``a`` followed by the ``nb`` rows of ``b`` (bf16 ``[..., n, C]``), and ``W`` is an fp32
per-token matrix.  One call is the read of a hyper-connection (``W`` = pre-weights ``[.., 1, n]``), another
its write-back (``W = [comb^T | post]`` over the streams and the sublayer output) - the forms of
``MHCConnection.prepare / combine`` (src/archlab/architectures/base.py:397-459) and of the V4.1 hyper
connection.  Backward: input gradients are the same kernel with ``W`` transposed, ``dW`` is a per-token
outer-product reduction.  Off the GPU an einsum runs.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import native

_vp, _i, _ll = C.c_void_p, C.c_int, C.c_longlong
native.register_signature("nga_token_mix", [_vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _vp])
native.register_signature("nga_token_mix_dw", [_vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _vp])
_OUTS = (1, 2, 3, 4, 5, 8)


def _p(t):
    return None if t is None else t.data_ptr()


def _usable(W, a, b):
    ni = a.size(-2) + (0 if b is None else b.size(-2))
    return (a.is_cuda and a.dtype == torch.bfloat16 and a.size(-1) % 8 == 0 and ni <= 8 and W.size(-2) in _OUTS
            and (b is None or b.dtype == torch.bfloat16) and native.available())


def _launch(a, b, W, n_out, transpose):
    tokens, na, C_ = a.numel() // (a.size(-2) * a.size(-1)), a.size(-2), a.size(-1)
    nb = 0 if b is None else b.size(-2)
    out = torch.empty(*a.shape[:-2], n_out, C_, dtype=a.dtype, device=a.device)
    native.check(native.lib().nga_token_mix(_p(a), _p(b), _p(W), _p(out), tokens, na, nb, n_out, C_, int(transpose),
                                            native.stream_ptr()), "nga_token_mix")
    return out


class _TokenMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, W, a, b):
        W32, a, b = W.float().contiguous(), a.contiguous(), None if b is None else b.contiguous()
        ctx.save_for_backward(W32, a, b)
        ctx.wdtype = W.dtype
        return _launch(a, b, W32, W.size(-2), False)

    @staticmethod
    def backward(ctx, dout):
        W32, a, b = ctx.saved_tensors
        dout = dout.contiguous()
        na, nb, no = a.size(-2), 0 if b is None else b.size(-2), W32.size(-2)
        ni = na + nb
        # d rows = W^T dout: one launch with `dout` as the input rows and the stored W read transposed
        if ni in _OUTS:
            drows = _launch(dout, None, W32, ni, True)
        else:
            drows = torch.einsum("...oj,...oc->...jc", W32, dout.float()).to(a.dtype)
        tokens = a.numel() // (na * a.size(-1))
        dW = torch.empty_like(W32)
        native.check(native.lib().nga_token_mix_dw(_p(dout), _p(a), _p(b), _p(dW), tokens, na, nb, no, a.size(-1),
                                                   native.stream_ptr()), "nga_token_mix_dw")
        da = drows[..., :na, :]
        db = None if b is None else drows[..., na:, :]
        return dW.to(ctx.wdtype), da, db


def token_mix(W: torch.Tensor, a: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    if _usable(W, a, b):
        return _TokenMix.apply(W, a, b)
    rows = a if b is None else torch.cat([a, b], -2)
    return torch.einsum("...oj,...jc->...oc", W.float(), rows.float()).to(a.dtype)


def hyper_connection_read(pre: torch.Tensor, streams: torch.Tensor) -> torch.Tensor:
    """pre [..., n], streams [..., n, C] -> sublayer input [..., C]."""
    return token_mix(pre.unsqueeze(-2), streams).squeeze(-2)


def hyper_connection_write(comb: torch.Tensor, post: torch.Tensor, streams: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """new_streams = comb^T streams + post (x) y.  comb [..., n, n], post [..., n], y [..., C]."""
    W = torch.cat([comb.transpose(-1, -2), post.unsqueeze(-1)], -1)
    return token_mix(W, streams, y.unsqueeze(-2))


# ------------------------------------------------------------------------------------------------
# hyper-connection coefficients (sigmoid read / write weights, Sinkhorn-balanced mixing matrix), n = 4
# ------------------------------------------------------------------------------------------------
_f = C.c_float
native.register_signature("nga_hc_coeff_fwd", [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _f, _vp])
native.register_signature("nga_hc_coeff_bwd", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _f, _vp])


class _HCCoeff(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mixes, scale, base, iters, eps):
        lead = mixes.shape[:-1]
        m = mixes.float().contiguous().view(-1, 24)
        T = m.size(0)
        sc, bs = scale.detach().float().contiguous(), base.detach().float().contiguous()
        pre = torch.empty(T, 4, dtype=torch.float32, device=m.device)
        post = torch.empty_like(pre)
        comb = torch.empty(T, 16, dtype=torch.float32, device=m.device)
        native.check(native.lib().nga_hc_coeff_fwd(_p(m), _p(sc), _p(bs), _p(pre), _p(post), _p(comb), T, 4, iters, eps,
                                                   native.stream_ptr()), "nga_hc_coeff_fwd")
        ctx.save_for_backward(m, sc, bs)
        ctx.meta = (lead, iters, eps, mixes.dtype, scale.dtype, base.dtype)
        return pre.view(*lead, 4), post.view(*lead, 4), comb.view(*lead, 4, 4)

    @staticmethod
    def backward(ctx, dpre, dpost, dcomb):
        m, sc, bs = ctx.saved_tensors
        lead, iters, eps, mdt, sdt, bdt = ctx.meta
        T = m.size(0)
        z = lambda g, n: (torch.zeros(T, n, dtype=torch.float32, device=m.device) if g is None else g.float().contiguous().view(T, n))
        dpre, dpost, dcomb = z(dpre, 4), z(dpost, 4), z(dcomb, 16)
        dm = torch.empty_like(m)
        dscale = torch.zeros(3, dtype=torch.float32, device=m.device)
        dbase = torch.zeros(24, dtype=torch.float32, device=m.device)
        native.check(native.lib().nga_hc_coeff_bwd(_p(m), _p(sc), _p(bs), _p(dpre), _p(dpost), _p(dcomb), _p(dm), _p(dscale), _p(dbase),
                                                   T, 4, iters, eps, native.stream_ptr()), "nga_hc_coeff_bwd")
        return dm.view(*lead, 24).to(mdt), dscale.to(sdt), dbase.to(bdt), None, None


def hc_coefficients_usable(mixes: torch.Tensor, streams: int, iterations: int) -> bool:
    return mixes.is_cuda and streams == 4 and 1 <= iterations <= 32 and mixes.dtype != torch.float64 and native.available()


def hc_coefficients(mixes, scale, base, iterations: int, eps: float):
    """mixes [..., 24] -> (pre [..., 4], post [..., 4], comb [..., 4, 4]) in fp32, one kernel each way."""
    return _HCCoeff.apply(mixes, scale, base, int(iterations), float(eps))
