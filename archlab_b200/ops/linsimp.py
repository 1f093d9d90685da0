"""LinSimp: linear-time 2-simplicial attention through positive orthogonal random features.

The long axis is summarised by causal prefix states of random features of the (L2-normalised) keys;
the short axis stays an explicit window of ``anchors`` r / u.  For query t and anchor c in the window
    w(t, c, j) ~ phi(tau * q_t * r_c) . phi(k_j),      out_t = sum_c u_c * (sum_j w v_j) / sum_c sum_j w
with phi(x) = m^-1/2 exp(Omega x - |x|^2 / 2) (src/archlab/architectures/linsimp_attention.py:36-176).
One shift per (query, head) over all anchors and features keeps the exponentials finite; it cancels
between numerator and denominator.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def orthogonal_feature_bank(heads: int, head_dim: int, rank: int, *, device=None, dtype=torch.float32, seed: int = 0):
    """[heads, rank, head_dim]: blocks of Haar-orthogonal directions scaled by chi_D radii."""
    if rank < 1 or rank % head_dim:
        raise ValueError("feature rank must be a positive multiple of head_dim")
    gen = torch.Generator().manual_seed(seed)
    blocks = []
    for _ in range(rank // head_dim):
        qf, rf = torch.linalg.qr(torch.randn(heads, head_dim, head_dim, generator=gen))
        sign = rf.diagonal(dim1=-2, dim2=-1).sign()
        sign = torch.where(sign == 0, torch.ones_like(sign), sign)
        dirs = (qf * sign.unsqueeze(-2)).transpose(-1, -2)
        radii = torch.randn(heads, head_dim, head_dim, generator=gen).norm(dim=-1)
        blocks.append(dirs * radii.unsqueeze(-1))
    return torch.cat(blocks, 1).to(device=device, dtype=dtype)


def positive_features(x, omega):
    sq = x.float().square().sum(-1, keepdim=True) * 0.5
    return (torch.einsum("...hd,hmd->...hm", x.float(), omega.float()) - sq).exp() * omega.shape[-2] ** -0.5


def _query_features(x, omega, anchor_axis=None, valid=None):
    logs = torch.einsum("...hd,hmd->...hm", x.float(), omega.float()) - x.float().square().sum(-1, keepdim=True) * 0.5
    if valid is not None:
        logs = logs.masked_fill(~valid[..., None, None], float("-inf"))
    axes = (-1,) if anchor_axis is None else (anchor_axis, -1)
    return (logs - logs.amax(axes, keepdim=True).detach()).exp() * omega.shape[-2] ** -0.5


def _unit(x, eps=1e-6):
    return x.float() / x.float().norm(dim=-1, keepdim=True).clamp_min(eps)


def _expand(q, *kv):
    rep = q.shape[2] // kv[0].shape[2]
    return [t.repeat_interleave(rep, 2) if rep > 1 else t for t in kv]


def linear_rf_attention(q, k, v, omega, *, temperature=None):
    """Causal one-mode random-feature attention (LinSimp without anchors)."""
    k, v = _expand(q, k, v)
    tau = math.sqrt(q.shape[-1]) if temperature is None else temperature
    qf = _query_features(_unit(q) * tau, omega)
    kf = positive_features(_unit(k), omega)
    state = (kf.unsqueeze(-1) * v.float().unsqueeze(-2)).cumsum(1)
    norm = kf.cumsum(1)
    num = torch.einsum("bthm,bthmd->bthd", qf, state)
    den = torch.einsum("bthm,bthm->bth", qf, norm).unsqueeze(-1).clamp_min(1e-30)
    return (num / den).to(q.dtype)


def linsimp_attention(q, k, r, v, u, omega, *, window: int, temperature=None):
    if r.shape != k.shape or u.shape != v.shape:
        raise ValueError("r/u must match k/v geometry")
    if window < 1:
        raise ValueError("anchor window must be a positive integer")
    k, r, v, u = _expand(q, k, r, v, u)
    B, T, H, D = q.shape
    tau = math.sqrt(D) if temperature is None else temperature
    qn, rn = _unit(q) * tau, _unit(r)
    kf = positive_features(_unit(k), omega)
    state = (kf.unsqueeze(-1) * v.float().unsqueeze(-2)).cumsum(1)
    norm = kf.cumsum(1)
    pad = window - 1
    win = lambda x: F.pad(x, (0, 0, 0, 0, pad, 0)).unfold(1, window, 1).permute(0, 1, 4, 2, 3)   # [B,T,W,H,D]
    rw, uw = win(rn), win(u.float())
    valid = torch.arange(window, device=q.device).view(1, 1, window) >= (pad - torch.arange(T, device=q.device)).clamp_min(0).view(1, T, 1)
    feat = _query_features(qn.unsqueeze(2) * rw, omega, anchor_axis=2, valid=valid)
    num = torch.einsum("btwhm,bthmd->btwhd", feat, state) * uw
    den = torch.einsum("btwhm,bthm->btwh", feat, norm)
    m = valid.to(num.dtype)
    num, den = num * m[..., None, None], den * m[..., None]
    return (num.sum(2) / den.sum(2).unsqueeze(-1).clamp_min(1e-30)).to(q.dtype)


def linsimp_attention_loop(q, k, r, v, u, omega, *, window: int, temperature=None):
    """Per-position loop; the parity oracle of the vectorised form."""
    k, r, v, u = _expand(q, k, r, v, u)
    tau = math.sqrt(q.shape[-1]) if temperature is None else temperature
    qn, rn = _unit(q) * tau, _unit(r)
    kf = positive_features(_unit(k), omega)
    state = (kf.unsqueeze(-1) * v.float().unsqueeze(-2)).cumsum(1)
    norm = kf.cumsum(1)
    outs = []
    for t in range(q.shape[1]):
        s = max(0, t - window + 1)
        feat = _query_features(qn[:, t].unsqueeze(1) * rn[:, s:t + 1], omega, anchor_axis=1)
        num = torch.einsum("bwhm,bhmd->bwhd", feat, state[:, t]) * u.float()[:, s:t + 1]
        den = torch.einsum("bwhm,bhm->bwh", feat, norm[:, t])
        outs.append(num.sum(1) / den.sum(1).unsqueeze(-1).clamp_min(1e-30))
    return torch.stack(outs, 1).to(q.dtype)
