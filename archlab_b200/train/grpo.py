"""GRPO policy update on token-level trajectories.

A group is the set of responses sampled for one prompt.  Advantages are the group-centred (optionally
std-normalised) scalar rewards, broadcast over the response tokens that the policy generated (tool
output tokens are masked out).  The loss is the clipped importance-weighted policy gradient with a hard
cap on the importance ratio (2.0: samples whose ratio exceeds it carry no gradient), no KL term, token-mean
over the batch - the science contract the experiment validators pin (GRPO only, IS cap 2.0, no KL;
src/archlab/training/config.py:149-229).  Groups whose rewards are all equal give no gradient and are
reported as wasted.  Log-probabilities come from the chunked head processor, so the [tokens, vocab]
logits never exist at once.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class GRPOConfig:
    clip_low: float = 0.2
    clip_high: float = 0.28
    is_cap: float = 2.0
    normalize_std: bool = True
    eps: float = 1e-6


def group_advantages(rewards: torch.Tensor, group_ids: torch.Tensor, cfg: GRPOConfig = GRPOConfig()):
    """rewards [N], group_ids [N] -> (advantages [N], informative mask [N]: groups with unequal rewards)."""
    adv = torch.zeros_like(rewards, dtype=torch.float32)
    informative = torch.zeros_like(rewards, dtype=torch.bool)
    for g in group_ids.unique():
        m = group_ids == g
        r = rewards[m].float()
        if r.numel() < 2:
            raise ValueError("every prompt needs at least two rollouts")
        centred = r - r.mean()
        spread = r.std(unbiased=False)
        if float(spread) > 0:
            adv[m] = centred / (spread + cfg.eps) if cfg.normalize_std else centred
            informative[m] = True
    return adv, informative


def grpo_loss(new_logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor,
              cfg: GRPOConfig = GRPOConfig()):
    """new/old log-probs [N, T] of the taken tokens, advantages [N], mask [N, T] (policy-generated tokens).
    Returns (loss, metrics)."""
    if new_logp.shape != old_logp.shape or mask.shape != new_logp.shape or advantages.shape != new_logp.shape[:1]:
        raise ValueError("misaligned trajectories")
    m = mask.float()
    n = m.sum().clamp_min(1.0)
    ratio = torch.exp(new_logp.float() - old_logp.float().detach())
    a = advantages.float().unsqueeze(1)
    unclipped = ratio * a
    clipped = torch.clamp(ratio, 1 - cfg.clip_low, 1 + cfg.clip_high) * a
    per_tok = -torch.minimum(unclipped, clipped)
    capped = ratio.detach() > cfg.is_cap                           # off-policy beyond the cap: no gradient at all
    per_tok = torch.where(capped, per_tok.detach(), per_tok)
    loss = (per_tok * m).sum() / n
    with torch.no_grad():
        metrics = {"clip_fraction": float((((ratio < 1 - cfg.clip_low) | (ratio > 1 + cfg.clip_high)).float() * m).sum() / n),
                   "cap_fraction": float((capped.float() * m).sum() / n),
                   "mean_ratio": float((ratio * m).sum() / n),
                   "policy_lag_kl": float(((old_logp.float() - new_logp.float()) * m).sum() / n)}
    return loss, metrics


def sequence_logprobs(model, ids: torch.Tensor, *, chunk_size: int = 512) -> torch.Tensor:
    """log pi(ids[:, t+1] | ids[:, :t+1]) for t = 0 .. T-2, through the model's hidden states and the
    chunked head (``model.hidden(ids)`` and ``model.lm_head``)."""
    from ..models.limite import chunked_logits_processor, logprob_entropy_processor

    h = model.hidden(ids)[:, :-1]
    out = chunked_logits_processor(model.lm_head, h, logprob_entropy_processor, {"labels": ids[:, 1:]}, chunk_size=chunk_size)
    return out["log_probs"]


def grpo_step(model, optimizer, batch: dict, cfg: GRPOConfig = GRPOConfig(), *, max_grad_norm: float = 1.0) -> dict:
    """batch: ids [N, T], old_logp [N, T-1], mask [N, T-1], rewards [N], group_ids [N], policy_version [N].
    One optimizer step; returns metrics including the wasted-group share."""
    adv, informative = group_advantages(batch["rewards"], batch["group_ids"], cfg)
    new_logp = sequence_logprobs(model, batch["ids"])
    loss, metrics = grpo_loss(new_logp, batch["old_logp"], adv.to(new_logp.device), batch["mask"], cfg)
    optimizer.zero_grad(set_to_none=True)
    loss.backward()
    gnorm = torch.nn.utils.clip_grad_norm_([p for p in model.parameters() if p.grad is not None], max_grad_norm)
    if not torch.isfinite(loss) or not torch.isfinite(gnorm):
        raise FloatingPointError("non-finite GRPO loss or gradient")
    optimizer.step()
    metrics.update(loss=float(loss.detach()), grad_norm=float(gnorm), wasted_group_share=1.0 - float(informative.float().mean()))
    return metrics
