"""Triadic gated delta network: a joint-key delta rule over ``E`` feature slices.

State ``S[e]`` (one ``[key_dim, value_dim]`` matrix per feature slice e).  Per token
    S[e] <- exp(g[e]) S[e]
    r     = v - sum_e k2[e] * (k^T S[e])                 (ONE residual erases the joint memory)
    S[e] <- S[e] + beta * k2[e] * (k r^T)
    o     = scale * sum_e q2[e] * (q^T S[e])
(src/archlab/architectures/triadic_attention.py:148-187; the incumbent is an external CuTe kernel).
Equivalently a delta rule on the joint key ``kron(k2, k)`` with per-slice decay, which is how the
chunked form below (and the sm_100a kernel design) treats it: the per-channel-decay KDA recurrence on
keys of width ``E * key_dim``.  Packed documents (``cu_seqlens``) reset the state at each boundary.
"""
from __future__ import annotations

import math

import torch

from . import delta_rule


def _check(q, k, v, k2, q2, g, beta):
    if q.ndim != 4 or min(q.shape) < 1:
        raise ValueError("q must be nonempty [batch, sequence, heads, key_dim]")
    B, T, H, _ = q.shape
    if k.shape != q.shape or v.ndim != 4 or v.shape[:3] != q.shape[:3]:
        raise ValueError("q/k must match and v must share batch/sequence/heads")
    if k2.ndim != 4 or k2.shape[:3] != (B, T, H) or k2.shape[-1] < 1:
        raise ValueError("k2 must be [batch, sequence, heads, feature_dim]")
    if q2.shape != k2.shape or g.shape != k2.shape or beta.shape != q.shape[:3]:
        raise ValueError("q2/g must match k2 and beta must be [batch, sequence, heads]")


def _segments(cu_seqlens, B, T):
    if cu_seqlens is None:
        return [0, T]
    offs = cu_seqlens.tolist()
    if B != 1 or len(offs) < 2 or offs[0] != 0 or offs[-1] != T or any(a >= b for a, b in zip(offs, offs[1:])):
        raise ValueError("document offsets must strictly increase from zero to sequence length (one packed row)")
    return offs


def triadic_gdn_reference(q, k, v, k2, q2, g, beta, *, scale=None, cu_seqlens=None):
    """Token-by-token recurrence (fp32, or fp64 when any input is fp64)."""
    _check(q, k, v, k2, q2, g, beta)
    B, T, H, D = q.shape
    starts = set(_segments(cu_seqlens, B, T)[:-1])
    dt = torch.float64 if any(t.dtype == torch.float64 for t in (q, k, v, k2, q2, g, beta)) else torch.float32
    out_dtype = q.dtype
    q, k, v, k2, q2, g, beta = (t.to(dt) for t in (q, k, v, k2, q2, g, beta))
    mult = D ** -0.5 if scale is None else scale
    if not math.isfinite(mult):
        raise ValueError("read scale must be finite")
    S = q.new_zeros(B, H, k2.size(-1), D, v.size(-1))
    outs = []
    for t in range(T):
        if t in starts:
            S = torch.zeros_like(S)
        S = S * g[:, t].exp()[..., None, None]
        pred = torch.einsum("bhd,bhedv,bhe->bhv", k[:, t], S, k2[:, t])
        r = v[:, t] - pred
        S = S + torch.einsum("bh,bhe,bhd,bhv->bhedv", beta[:, t], k2[:, t], k[:, t], r)
        outs.append(mult * torch.einsum("bhd,bhedv,bhe->bhv", q[:, t], S, q2[:, t]))
    return torch.stack(outs, 1).to(out_dtype)


def triadic_gdn_chunked(q, k, v, k2, q2, g, beta, *, scale=None, cu_seqlens=None, chunk: int = 64):
    """Chunk-parallel form through the joint key ``kron(k2, k)``: per-channel-decay delta rule."""
    _check(q, k, v, k2, q2, g, beta)
    B, T, H, D = q.shape
    E = k2.size(-1)
    mult = D ** -0.5 if scale is None else scale
    jk = (k2.float().unsqueeze(-1) * k.float().unsqueeze(-2)).flatten(-2)          # [B,T,H,E*D]
    jq = (q2.float().unsqueeze(-1) * q.float().unsqueeze(-2)).flatten(-2)
    jg = g.float().unsqueeze(-1).expand(B, T, H, E, D).flatten(-2)
    offs = _segments(cu_seqlens, B, T)
    outs = []
    for a, b in zip(offs, offs[1:]):
        outs.append(_raw_delta(jq[:, a:b], jk[:, a:b], v[:, a:b].float(), jg[:, a:b], beta[:, a:b].float(), chunk))
    return (mult * torch.cat(outs, 1)).to(q.dtype)


def _raw_delta(q, k, v, g, beta, chunk):
    """``delta_rule.chunk_kda`` without its q/k normalisation (the triadic keys are used as given)."""
    saved = delta_rule._prep
    try:
        delta_rule._prep = lambda q, k, v, g, beta: (q.float(), k.float(), v.float(), g.float(), beta.float())
        return delta_rule.chunk_kda(q, k, v, g, beta, chunk=chunk)
    finally:
        delta_rule._prep = saved


def triadic_gdn_attention(q, k, v, k2, q2, g, beta, *, backend: str = "chunked", scale=None, cu_seqlens=None):
    if backend == "reference":
        return triadic_gdn_reference(q, k, v, k2, q2, g, beta, scale=scale, cu_seqlens=cu_seqlens)
    if backend != "chunked":
        raise ValueError("Triadic backend must be chunked or reference")
    return triadic_gdn_chunked(q, k, v, k2, q2, g, beta, scale=scale, cu_seqlens=cu_seqlens)
