"""DeepSeek sparse attention (DSA): lightning indexer -> top-k key selection -> gathered attention
with a per-head sink logit, plus the indexer's KL objective.

* ``indexer_scores``: weighted-ReLU multi-query scores ``sum_h w[t,h] relu(q[t,h] . k[s]) * scale``
  with a causal mask (src/archlab/architectures/dsa.py:85-233).
* ``select_topk``: top-k keys per query; slots that fall on masked keys are returned as ``-1``.
* ``sparse_attention``: queries [B,S,H,D] attend to rows of a shared latent KV [B,K,D] gathered
  by indices [B,S,T]; the sink adds denominator-only mass; repeated slots count each time; the
  ``native_rounding`` mode rounds un-normalised exponentials to bf16 in 64-key blocks with an fp32
  denominator (src/archlab/architectures/deepseek_v41_torch.py:16-78).
* ``indexer_kl``: KL(main attention averaged over heads || softmax(index scores)) over the valid set
  (src/archlab/architectures/deepseek_v41_indexer_objective.py:5-24, dsa.py:129-233).

These are the fp32 oracles of the sm_100a DSA kernels and the CPU / fallback path.
"""
from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint


def indexer_scores(q: torch.Tensor, k: torch.Tensor, weights: torch.Tensor, scale: float | None = None,
                   *, query_offset: int = 0, positions: torch.Tensor | None = None) -> torch.Tensor:
    """q [B,S,Hi,Di], k [B,K,Di], weights [B,S,Hi] -> scores [B,S,K] (fp32, -inf above the diagonal).
    Query i sits at absolute position ``query_offset + i`` (or ``positions[i]`` when given)."""
    scale = q.size(-1) ** -0.5 if scale is None else scale
    per_head = torch.einsum("bqhd,bkd->bqhk", q.float(), k.float()).relu()
    s = (per_head * weights.float().unsqueeze(-1)).sum(2) * scale
    qpos = torch.arange(q.size(1), device=q.device) + query_offset if positions is None else positions
    kpos = torch.arange(k.size(1), device=q.device)
    return s.masked_fill(kpos[None, None, :] > qpos[None, :, None], float("-inf"))


def select_topk(scores: torch.Tensor, top_k: int):
    """-> (indices [B,S,min(k,K)] int64 with -1 for slots on masked keys, selected score values)."""
    k = min(top_k, scores.size(-1))
    vals, idx = scores.topk(k, dim=-1)
    return torch.where(torch.isfinite(vals), idx, torch.full_like(idx, -1)), vals


def _sparse_chunk(q, kv, sink, indices, scale, native_rounding):
    dt = torch.float64 if q.dtype == torch.float64 else torch.float32
    K = kv.size(1)
    valid = (indices >= 0) & (indices < K)
    safe = indices.clamp(0, max(K - 1, 0)).long()
    rows = kv[torch.arange(q.size(0), device=q.device)[:, None, None], safe].to(dt)           # [B,S,T,D]
    scores = torch.einsum("bshd,bstd->bsht", q.to(dt), rows) * scale
    scores = scores.masked_fill(~valid.unsqueeze(2), float("-inf"))
    sinks = sink.to(dt)[None, None, :, None]
    if not native_rounding:
        p = torch.cat([scores, sinks.expand(*scores.shape[:-1], 1)], -1).softmax(-1)[..., :-1]
        return torch.einsum("bsht,bstd->bshd", p, rows).to(q.dtype)
    m = scores.new_full((*scores.shape[:-1], 1), -1e30)
    den = torch.zeros_like(m)
    num = torch.zeros(q.shape, dtype=dt, device=q.device)
    for t0 in range(0, scores.size(-1), 64):
        blk = scores[..., t0:t0 + 64]
        m2 = torch.maximum(m, blk.amax(-1, keepdim=True))
        r = torch.exp(m - m2)
        e = torch.exp(blk - m2)
        den = den * r + e.sum(-1, keepdim=True)
        num = num * r + torch.einsum("bsht,bstd->bshd", e.to(torch.bfloat16).to(dt), rows[:, :, t0:t0 + 64])
        m = m2
    top = torch.maximum(m, sinks)
    r = torch.exp(m - top)
    return (num * r / (den * r + torch.exp(sinks - top))).to(q.dtype)


def sparse_attention(q: torch.Tensor, kv: torch.Tensor, sink: torch.Tensor, indices: torch.Tensor, scale: float, *,
                     query_chunk: int = 32, recompute: bool = True, native_rounding: bool = False) -> torch.Tensor:
    if query_chunk < 1 or q.ndim != 4 or kv.ndim != 3 or indices.ndim != 3:
        raise ValueError("invalid sparse attention geometry")
    if q.shape[:2] != indices.shape[:2] or q.shape[0] != kv.shape[0] or q.shape[-1] != kv.shape[-1]:
        raise ValueError("mismatched sparse attention tensors")
    if sink.shape != (q.shape[2],) or kv.shape[1] < 1 or q.shape[1] < 1:
        raise ValueError("empty KV/query or invalid sink")
    outs = []
    for s0 in range(0, q.size(1), query_chunk):
        args = (q[:, s0:s0 + query_chunk], kv, sink, indices[:, s0:s0 + query_chunk], scale, native_rounding)
        if recompute and torch.is_grad_enabled() and any(t.requires_grad for t in (q, kv, sink)):
            outs.append(checkpoint(_sparse_chunk, *args, use_reentrant=False))
        else:
            outs.append(_sparse_chunk(*args))
    return torch.cat(outs, 1)


def dense_sink_attention(q: torch.Tensor, kv: torch.Tensor, sink: torch.Tensor, scale: float) -> torch.Tensor:
    """All causal keys (the dense warm-up phase / the k >= K limit of ``sparse_attention``)."""
    S, K = q.size(1), kv.size(1)
    s = torch.einsum("bshd,bkd->bshk", q.float(), kv.float()) * scale
    mask = torch.arange(K, device=q.device)[None, :] > (torch.arange(S, device=q.device)[:, None] + (K - S))
    s = s.masked_fill(mask[None, :, None, :], float("-inf"))
    p = torch.cat([s, sink.float()[None, None, :, None].expand(*s.shape[:-1], 1)], -1).softmax(-1)[..., :-1]
    return torch.einsum("bshk,bkd->bshd", p, kv.float()).to(q.dtype)


def indexer_kl(target: torch.Tensor, index_scores: torch.Tensor, valid: torch.Tensor) -> torch.Tensor:
    """KL(target || softmax(index_scores)) over ``valid`` slots, averaged over queries that have any."""
    logp = index_scores.masked_fill(~valid, float("-inf")).log_softmax(-1)
    t = target.masked_fill(~valid, 0.0)
    t = t / t.sum(-1, keepdim=True).clamp_min(1e-20)
    terms = torch.where(valid & (t > 0), t * (t.clamp_min(1e-30).log() - logp), torch.zeros_like(t))
    has = valid.any(-1)
    return (terms.sum(-1) * has).sum() / has.sum().clamp_min(1)


def main_attention_target(main_q: torch.Tensor, kv: torch.Tensor, scale: float, positions: torch.Tensor | None = None) -> torch.Tensor:
    """Head-averaged causal softmax of the main attention (detached) -> [B,S,K].  ``positions`` [S] gives the
    absolute position of every query row when only a subset of the rows is passed."""
    S, K = main_q.size(1), kv.size(1)
    s = torch.einsum("bshd,bkd->bhsk", main_q.detach().float(), kv.detach().float()) * scale
    qpos = torch.arange(S, device=s.device) + (K - S) if positions is None else positions
    mask = torch.arange(K, device=s.device)[None, :] > qpos[:, None]
    return s.masked_fill(mask, float("-inf")).softmax(-1).mean(1)


def kl_rows(S: int, max_rows: int, step: int, device) -> torch.Tensor | None:
    """Query rows on which the indexer's KL is evaluated: all of them up to ``max_rows``, else a strided subset whose
    offset moves with the training step so that every row is visited."""
    if max_rows <= 0 or S <= max_rows:
        return None
    stride = (S + max_rows - 1) // max_rows
    return torch.arange(step % stride, S, stride, device=device)
