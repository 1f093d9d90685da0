"""Two loss-normalisation contracts that must not be mixed: the mean over equally sized components, and the mean over
the GLOBAL number of supervised tokens.

With masked labels (SFT, packed documents, multi-token prediction) micro-batches and ranks hold different numbers of
supervised tokens, so averaging per micro-batch means weights tokens of sparse batches more.  The per-token contract
returns ``(loss_sum, token_count)`` from every micro-batch and divides once, by the token count of the whole step over
all ranks.  Auxiliary losses (router balance, z-loss, MTP) are per-token sums as well and divide by the same count, so
their weight relative to the language-model loss does not depend on how the batch was cut.

* ``component_mean_loss(losses, metrics)``      the legacy contract: mean over elements, metrics as (value, 1) pairs;
* ``masked_token_loss(loss_mask, losses)``       (sum, count, report) of one micro-batch;
* ``TokenNormalizedStep``                        accumulates micro-batches: ``backward(loss_sum, count)`` back-propagates
  the SUM, ``finish(parameters, group)`` all-reduces the count and scales every gradient by ``world / global_tokens``
  when gradients are averaged over ranks afterwards (or ``1 / global_tokens`` when they are summed).
(Reference: src/archlab/megatron/losses.py:10-47.)
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def component_mean_loss(losses: torch.Tensor, component_metrics: dict[str, torch.Tensor] | None = None):
    flat = losses.reshape(-1).float()
    count = torch.tensor(float(flat.numel()), device=flat.device)
    total = flat.sum()
    report = {"lm loss": torch.stack((total.detach(), count))}
    for name, value in (component_metrics or {}).items():
        report[name] = torch.stack((value.detach().float(), torch.ones((), device=value.device)))
    return total / count, report


def masked_token_loss(loss_mask: torch.Tensor, losses: torch.Tensor):
    flat, mask = losses.reshape(-1).float(), loss_mask.reshape(-1).float()
    total = (flat * mask).sum()
    count = mask.sum().to(torch.int64)
    return total, count, {"lm loss": torch.stack((total.detach(), count.float()))}


class TokenNormalizedStep:
    def __init__(self):
        self.tokens = None
        self.loss_sum = None

    def backward(self, loss_sum: torch.Tensor, count: torch.Tensor, *auxiliary_sums: torch.Tensor) -> None:
        """Back-propagates the un-normalised sums of one micro-batch (language-model loss plus per-token auxiliary sums)."""
        total = loss_sum + sum(auxiliary_sums) if auxiliary_sums else loss_sum
        total.backward()
        self.tokens = count.detach().clone() if self.tokens is None else self.tokens + count.detach()
        self.loss_sum = loss_sum.detach().clone() if self.loss_sum is None else self.loss_sum + loss_sum.detach()

    def finish(self, parameters, group=None, *, gradients_are_averaged: bool = True) -> dict:
        """Call after the last micro-batch and BEFORE the gradient all-reduce.  Returns the step's mean loss."""
        if self.tokens is None:
            raise RuntimeError("no micro-batch was accumulated")
        tokens, loss = self.tokens.clone().float(), self.loss_sum.clone().float()
        world = 1
        if dist.is_available() and dist.is_initialized():
            world = dist.get_world_size(group)
            packed = torch.stack((tokens, loss))
            dist.all_reduce(packed, group=group)
            tokens, loss = packed[0], packed[1]
        if float(tokens) <= 0:
            raise RuntimeError("the step holds no supervised token")
        scale = (world if gradients_are_averaged else 1) / float(tokens)
        for p in parameters:
            if p.grad is not None:
                p.grad.mul_(scale)
        self.tokens = self.loss_sum = None
        return {"loss": float(loss / tokens), "global_tokens": int(tokens), "gradient_scale": scale}
