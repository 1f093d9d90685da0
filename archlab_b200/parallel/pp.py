"""Pipeline parallelism: contiguous layer stages, one-forward-one-backward schedule over point-to-point
transfers.

A stage owns a slice of the layer stack.  Activations travel to the next stage and their gradients back
with ``torch.distributed`` point-to-point operations; whenever a stage has both something to send and
something to receive with the same neighbour the two go into ONE ``batch_isend_irecv`` group, so that
neither side can block the other (NCCL runs grouped sends and receives as one kernel; gloo completes
them independently).  In-flight activations per stage are bounded by ``n_stages - stage`` micro-batches.

Takes the place of Megatron's pipeline schedule used by the reference's mesh launches
(``qwen38_flash_next_config.py:205-221`` passes ``--pipeline-model-parallel-size``); the schedule is
the usual warm-up / steady one-forward-one-backward / cool-down order.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Sequence

import torch
import torch.distributed as dist


def split_layers(n_layers: int, n_stages: int) -> list[range]:
    """Contiguous, as-even-as-possible layer ranges; earlier stages take the remainder."""
    if not 1 <= n_stages <= n_layers:
        raise ValueError("need 1 <= stages <= layers")
    base, extra = divmod(n_layers, n_stages)
    out, start = [], 0
    for s in range(n_stages):
        n = base + (1 if s < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


@dataclass
class StageLinks:
    stage: int
    n_stages: int
    prev_rank: int | None          # global ranks of the neighbours (None at the ends)
    next_rank: int | None
    group: object = None

    @property
    def first(self) -> bool:
        return self.stage == 0

    @property
    def last(self) -> bool:
        return self.stage == self.n_stages - 1


def _exchange(links: StageLinks, *, send_next=None, send_prev=None, recv_next=None, recv_prev=None) -> None:
    ops = []
    if send_prev is not None:
        ops.append(dist.P2POp(dist.isend, send_prev, links.prev_rank, links.group))
    if recv_prev is not None:
        ops.append(dist.P2POp(dist.irecv, recv_prev, links.prev_rank, links.group))
    if send_next is not None:
        ops.append(dist.P2POp(dist.isend, send_next, links.next_rank, links.group))
    if recv_next is not None:
        ops.append(dist.P2POp(dist.irecv, recv_next, links.next_rank, links.group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


def run_1f1b(links: StageLinks, stage_fn: Callable, microbatches: Sequence, *, act_shape, act_dtype, device,
             loss_scale: float = 1.0) -> torch.Tensor:
    """Run one optimizer step's micro-batches through this stage.

    ``stage_fn(x_or_none, microbatch)`` returns the stage's output activation, or on the last stage the
    scalar loss of that micro-batch; on the first stage ``x_or_none`` is None and the stage reads its
    input from the micro-batch.  Returns the summed (scaled) loss on the last stage, zero elsewhere.
    Gradients accumulate into the stage's parameters.
    """
    n = len(microbatches)
    warm = min(links.n_stages - links.stage - 1, n)
    steady = n - warm
    pending: list[tuple[torch.Tensor | None, torch.Tensor]] = []
    total = torch.zeros((), device=device)
    fwd_i = 0

    def new_buf():
        return torch.empty(act_shape, dtype=act_dtype, device=device)

    def forward(x_in):
        nonlocal fwd_i, total
        if x_in is not None:
            x_in.requires_grad_(True)
        out = stage_fn(x_in, microbatches[fwd_i])
        fwd_i += 1
        if links.last:
            out = out * loss_scale
            total = total + out.detach()
        pending.append((x_in, out))
        return out

    def backward(grad_out):
        x_in, out = pending.pop(0)
        if links.last:
            out.backward()
        else:
            out.backward(grad_out)
        return None if x_in is None else x_in.grad

    x = None
    for _ in range(warm):
        if not links.first:
            x = new_buf()
            _exchange(links, recv_prev=x)
        out = forward(x)
        if not links.last:
            _exchange(links, send_next=out.detach().contiguous())
    if steady and not links.first:
        x = new_buf()
        _exchange(links, recv_prev=x)
    for i in range(steady):
        out = forward(x if not links.first else None)
        g = None
        if not links.last:
            g = new_buf()
            _exchange(links, send_next=out.detach().contiguous(), recv_next=g)
        gx = backward(g)
        more = i + 1 < steady
        x = new_buf() if (more and not links.first) else None
        if not links.first:
            _exchange(links, send_prev=gx.contiguous(), recv_prev=x)
    for _ in range(warm):
        g = None
        if not links.last:
            g = new_buf()
            _exchange(links, recv_next=g)
        gx = backward(g)
        if not links.first:
            _exchange(links, send_prev=gx.contiguous())
    return total
