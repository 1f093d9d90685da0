"""Distributed qualification checks of a sharded model, independent of any trainer: how many UNIQUE parameters the job
holds, and whether tensors that are supposed to be replicas really are equal after optimizer steps.

* ``unique_parameter_counts``: every rank sums its dense parameters (replicated over the data-parallel replicas) and its
  expert-side parameters (marked ``allreduce = False``: experts, owner-sharded tables; replicated over the expert-data-
  parallel replicas only); the all-reduced totals must divide by the replica counts, and the quotients are the model's
  unique parameter counts -- to be compared with the closed-form contract.
* ``replica_equality``: for every parameter selected by name, the first rank of the replica group broadcasts its tensor
  and every rank compares bit for bit (non-finite values count as mismatches); no selected parameter at all is an error
  too, so a renamed module cannot make the check pass vacuously.
* ``effective_gradient``: a fused weight-gradient kernel that accumulates straight into the main-gradient buffer leaves
  a placeholder in ``.grad``; the check reads the buffer then.
(Reference: src/archlab/megatron/qwen38_flash_next_checks.py:8-80.)
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def unique_parameter_counts(model, *, data_replicas: int, expert_replicas: int, group=None) -> dict:
    counts = [0, 0]
    for p in model.parameters():
        counts[int(not getattr(p, "allreduce", True))] += p.numel()
    device = next(model.parameters()).device
    totals = torch.tensor(counts, dtype=torch.int64, device=device)
    if dist.is_initialized():
        dist.all_reduce(totals, group=group)
    dense, expert = totals.tolist()
    if dense % data_replicas or expert % expert_replicas:
        raise RuntimeError("parameters do not divide into complete model replicas")
    return {"dense_unique": dense // data_replicas, "expert_side_unique": expert // expert_replicas,
            "total": dense // data_replicas + expert // expert_replicas}


def replica_equality(model, replica_group, name_parts: tuple[str, ...]) -> dict:
    """``replica_group``: the ranks that hold copies of the same shard (None: all ranks)."""
    source = dist.get_process_group_ranks(replica_group)[0] if replica_group is not None else 0
    checked, bad = 0, None
    for name, p in model.named_parameters():
        if not any(part in name for part in name_parts):
            continue
        bad = torch.zeros((), dtype=torch.int64, device=p.device) if bad is None else bad
        reference = p.detach().clone()
        dist.broadcast(reference, src=source, group=replica_group)
        bad += ((p.detach() != reference) | ~torch.isfinite(p.detach())).any().to(torch.int64)
        checked += 1
    device = next(model.parameters()).device
    evidence = torch.stack(((bad if bad is not None else torch.zeros((), dtype=torch.int64, device=device)),
                            torch.tensor(checked, dtype=torch.int64, device=device)))
    dist.all_reduce(evidence)
    if evidence[0].item() or not evidence[1].item():
        raise RuntimeError(f"replica equality failed: mismatching ranks-tensors {evidence[0].item()}, checked {evidence[1].item()}")
    return {"status": "passed", "checked_tensors_all_ranks": int(evidence[1].item()), "mismatches": 0}


def effective_gradient(parameter, autograd_gradient):
    if getattr(parameter, "grad_added_to_main_grad", False):
        return parameter.main_grad
    return autograd_gradient
