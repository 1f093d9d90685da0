"""Causal local 2-simplicial (trilinear) attention.

For query i, with a short window of ``w1`` positions ``j in (i-w1, i]`` carrying (k1, v1) and a long
window of ``w2`` positions ``k in (i-w2, i]`` carrying (k2, v2):

    s[j, k] = scale * sum_d q[i, d] * k1[j, d] * k2[k, d]
    p       = softmax over ALL causal (j, k) pairs jointly
    out[i]  = sum_{j,k} p[j, k] * (v1[j] * v2[k])

Layout ``[batch, sequence, heads, head_dim]``, grouped-query: q may have a multiple of the k/v
heads.  This is the semantics of the reference oracle
(src/archlab/architectures/simplicial_attention.py:49-74) and of its Triton / TileLang kernels
(simplicial_kernels.py:16-106, tilelang_attention.py:25-263).

``simplicial_attention_reference`` is a vectorised, differentiable PyTorch statement (query-chunked
so it never builds an N x w1 x w2 tensor for the whole sequence); it is the CPU path and the oracle
for the sm_100a kernel in ``csrc/simplicial.cu`` that ``simplicial_attention`` dispatches to on CUDA.
"""
from __future__ import annotations

import math

import torch


def validate_inputs(q, k1, k2, v1, v2, w1: int, w2: int) -> None:
    if q.ndim != 4 or any(x.ndim != 4 for x in (k1, k2, v1, v2)):
        raise ValueError("expected [batch, sequence, heads, head_dim]")
    if min(w1, w2) < 1 or w1 > w2:
        raise ValueError("require 1 <= short_window <= long_window")
    b, n, h, d = q.shape
    if min(b, n, h, d) < 1:
        raise ValueError("empty attention dimensions are unsupported")
    if k2.shape != k1.shape or v2.shape != v1.shape or v1.shape[:3] != k1.shape[:3]:
        raise ValueError("both key/value branches must have matching batch, sequence and heads")
    if k1.shape[:2] != (b, n) or k1.shape[-1] != d or h % k1.shape[2]:
        raise ValueError("incompatible grouped-query geometry")
    if any(x.dtype != q.dtype or x.device != q.device for x in (k1, k2, v1, v2)):
        raise ValueError("all inputs must have the same dtype and device")


def _window_gather(x: torch.Tensor, start: int, stop: int, w: int):
    """x [B, N, H, D] -> windows [B, n, w, H, D] for queries start..stop-1 and the validity mask
    [n, w]; slot a of query i is position i - w + 1 + a."""
    i = torch.arange(start, stop, device=x.device).view(-1, 1)
    a = torch.arange(w, device=x.device).view(1, -1)
    pos = i - w + 1 + a
    valid = pos >= 0
    return x[:, pos.clamp_min(0)], valid


def simplicial_attention_reference(q, k1, k2, v1, v2, w1: int, w2: int, *, scale: float | None = None,
                                   query_chunk: int = 128) -> torch.Tensor:
    validate_inputs(q, k1, k2, v1, v2, w1, w2)
    B, N, H, D = q.shape
    g = H // k1.shape[2]
    if g > 1:
        k1, k2, v1, v2 = (x.repeat_interleave(g, dim=2) for x in (k1, k2, v1, v2))
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    outs = []
    for s in range(0, N, query_chunk):
        e = min(N, s + query_chunk)
        k1w, m1 = _window_gather(k1, s, e, w1)      # [B, n, w1, H, D]
        k2w, m2 = _window_gather(k2, s, e, w2)
        v1w, _ = _window_gather(v1, s, e, w1)
        v2w, _ = _window_gather(v2, s, e, w2)
        a = q[:, s:e].unsqueeze(2) * k1w           # [B, n, w1, H, D]
        sc = torch.einsum("bnahd,bnchd->bnhac", a, k2w) * scale
        mask = (m1.unsqueeze(-1) & m2.unsqueeze(-2)).view(1, e - s, 1, w1, w2)
        sc = sc.masked_fill(~mask, float("-inf"))
        p = sc.flatten(-2).softmax(-1).view_as(sc)
        # out = sum_a v1[a] * (sum_c p[a, c] v2[c])
        pv2 = torch.einsum("bnhac,bnchd->bnahd", p, v2w)
        outs.append((pv2 * v1w).sum(dim=2))
    return torch.cat(outs, dim=1)


def simplicial_attention(q, k1, k2, v1, v2, w1: int, w2: int, *, scale: float | None = None):
    """Dispatch: sm_100a kernel for CUDA bf16 inputs with head_dim 128 (forward and backward),
    otherwise the differentiable PyTorch statement above."""
    validate_inputs(q, k1, k2, v1, v2, w1, w2)
    if q.device.type == "cuda" and q.dtype == torch.bfloat16 and q.shape[-1] == 128:
        from .simplicial_cuda import SimplicialFunction, kernel_supports

        if kernel_supports(q, k1, v1, w1, w2):
            return SimplicialFunction.apply(q, k1, k2, v1, v2, w1, w2,
                                            1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale))
    return simplicial_attention_reference(q, k1, k2, v1, v2, w1, w2, scale=scale)


# ------------------------------------------------------------------------------------------------
# Determinant (Sarrus) variant: scores are sums of 3x3 determinants over coordinate triples
# (src/archlab/architectures/simplicial_attention.py:100-202).
# ------------------------------------------------------------------------------------------------
def determinant_operands(q, k1, k2):
    """Rewrite det-scores as two trilinear forms: returns (q_cat, k1_cat, k2_cat) with doubled
    width such that sum_d q_cat*k1_cat*k2_cat = sum over triples of det[q; k1; k2]."""
    D = q.shape[-1]
    if D < 3:
        raise ValueError("determinant scores require at least 3 coordinates")
    used = 3 * (D // 3)
    base = torch.arange(0, used, 3, device=q.device)[:, None]
    s1 = (base + torch.tensor([1, 2, 0], device=q.device)).flatten()
    s2 = (base + torch.tensor([2, 0, 1], device=q.device)).flatten()
    qq = q[..., :used]
    # det = sum_c q_c (k1_{c+1} k2_{c+2} - k1_{c+2} k2_{c+1})
    q_cat = torch.cat([qq, -qq], dim=-1)
    k1_cat = torch.cat([k1[..., s1], k1[..., s2]], dim=-1)
    k2_cat = torch.cat([k2[..., s2], k2[..., s1]], dim=-1)
    return q_cat, k1_cat, k2_cat


def determinant_simplicial_attention(q, k1, k2, v1, v2, w1: int, w2: int, *, scale: float | None = None):
    D = q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    qc, k1c, k2c = determinant_operands(q, k1, k2)
    B, N, H, _ = qc.shape
    g = H // k1.shape[2]
    if g > 1:
        k1c, k2c, v1, v2 = (x.repeat_interleave(g, dim=2) for x in (k1c, k2c, v1, v2))
    outs = []
    for s in range(0, N, 128):
        e = min(N, s + 128)
        k1w, m1 = _window_gather(k1c, s, e, w1)
        k2w, m2 = _window_gather(k2c, s, e, w2)
        v1w, _ = _window_gather(v1, s, e, w1)
        v2w, _ = _window_gather(v2, s, e, w2)
        a = qc[:, s:e].unsqueeze(2) * k1w
        sc = torch.einsum("bnahd,bnchd->bnhac", a, k2w) * scale
        mask = (m1.unsqueeze(-1) & m2.unsqueeze(-2)).view(1, e - s, 1, w1, w2)
        sc = sc.masked_fill(~mask, float("-inf"))
        p = sc.flatten(-2).softmax(-1).view_as(sc)
        pv2 = torch.einsum("bnhac,bnchd->bnahd", p, v2w)
        outs.append((pv2 * v1w).sum(dim=2))
    return torch.cat(outs, dim=1)
