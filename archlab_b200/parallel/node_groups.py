"""Process groups that must not leave a node.

Expert-parallel dispatch / combine and the fused tensor-parallel kernels here move data through NVLink peer memory, which
exists only between GPUs of one host; a group of consecutive ranks that straddles two hosts would silently fall off
that path (or, for symmetric-memory kernels, fail at the first access).  ``node_local_groups(size)`` gathers every rank's
host name, checks that each block of ``size`` consecutive ranks sits on ONE host, creates all groups on all ranks (group
creation is collective) and returns the caller's.  ``host_of`` is injectable so that the layout logic is testable on one
machine.  (Reference: src/archlab/automodel/deepseek_v41_execution.py:41-56.)
"""
from __future__ import annotations

import socket
from typing import Callable

import torch.distributed as dist


def group_layout(hosts: list[str], size: int) -> list[list[int]]:
    """Consecutive rank blocks of ``size``; raises if the world is not divisible or a block spans hosts."""
    world = len(hosts)
    if size < 1 or world % size:
        raise ValueError(f"the group size {size} must divide the world size {world}")
    blocks = [list(range(first, first + size)) for first in range(0, world, size)]
    for ranks in blocks:
        names = {hosts[r] for r in ranks}
        if len(names) != 1:
            raise ValueError(f"ranks {ranks[0]}..{ranks[-1]} span hosts {sorted(names)}; such groups must be node-local")
    return blocks


def node_local_groups(size: int, *, host_of: Callable[[], str] = socket.gethostname):
    """-> (this rank's group, its ranks).  Collective: every rank must call it with the same ``size``."""
    world, rank = dist.get_world_size(), dist.get_rank()
    hosts: list = [None] * world
    dist.all_gather_object(hosts, host_of())
    mine = None
    for ranks in group_layout(hosts, size):
        group = dist.new_group(ranks)
        if rank in ranks:
            mine = (group, ranks)
    return mine


def ranks_per_host(hosts: list[str]) -> dict[str, list[int]]:
    out: dict[str, list[int]] = {}
    for rank, host in enumerate(hosts):
        out.setdefault(host, []).append(rank)
    return out
