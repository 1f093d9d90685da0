"""Backend-portable collective helpers.

NCCL provides every primitive natively.  gloo (the CPU test backend) lacks
``reduce_scatter_tensor``, so that one is expressed as all-reduce + slice there; the semantics
(averaging, contiguous rank-major chunks along dim 0) are identical, which is what lets the
2-rank gloo tests exercise the same optimizer and engine code that runs over NVLink.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized()


def world_size(group=None) -> int:
    return dist.get_world_size(group) if is_dist() else 1


def rank(group=None) -> int:
    return dist.get_rank(group) if is_dist() else 0


def get_dist_info() -> tuple[bool, int, int, int]:
    """(distributed requested, rank, local rank, world size) from the torchrun environment
    (src/archlab/distributed.py:8-34)."""
    if all(k in os.environ for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE")):
        return True, int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    return False, 0, 0, 1


def _backend(group=None) -> str:
    return dist.get_backend(group)


class _Done:
    def wait(self):
        return None


def reduce_scatter_avg(out: torch.Tensor, inp: torch.Tensor, group=None, async_op: bool = False):
    """out = mean over ranks of inp's chunk ``rank`` along dim 0 (inp has world * out rows)."""
    ws = world_size(group)
    if ws == 1:
        out.copy_(inp)
        return _Done()
    if _backend(group) == "nccl":
        return dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.AVG, group=group, async_op=async_op) or _Done()
    tmp = inp.clone()
    dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
    r = rank(group)
    n = out.size(0)
    out.copy_(tmp[r * n:(r + 1) * n] / ws)
    return _Done()


def all_reduce_avg(t: torch.Tensor, group=None, async_op: bool = False):
    ws = world_size(group)
    if ws == 1:
        return _Done()
    if _backend(group) == "nccl":
        return dist.all_reduce(t, op=dist.ReduceOp.AVG, group=group, async_op=async_op) or _Done()
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    t.div_(ws)
    return _Done()


def all_gather_into(out: torch.Tensor, inp: torch.Tensor, group=None, async_op: bool = False):
    ws = world_size(group)
    if ws == 1:
        out.copy_(inp)
        return _Done()
    if _backend(group) == "nccl":
        return dist.all_gather_into_tensor(out, inp, group=group, async_op=async_op) or _Done()
    parts = list(out.chunk(ws, dim=0))
    dist.all_gather(parts, inp.contiguous(), group=group)
    return _Done()


def all_reduce_max_scalar(value: float, device, group=None) -> float:
    t = torch.tensor([value], dtype=torch.float32, device=device)
    if is_dist():
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
