"""ZeRO-style distributed Muon + AdamW (gradient sync lives inside the optimizer, no DDP wrapper).

Behaviour follows the reference's ``DistMuonAdamW`` (src/archlab/optimizers/speedrun.py:447-755):

* AdamW parameters with >= 1024 elements and a leading dimension divisible by the world size are
  reduce-scattered (mean) along dim 0; each rank updates its row slice (optimizer state exists only
  for the slice) and the slices are all-gathered back; small parameters are all-reduced and updated
  redundantly.
* Muon groups stack their K same-shape matrices, pad K up to a multiple of the world size,
  reduce-scatter so that each rank owns ``ceil(K / world)`` whole matrices, run the Muon update on
  the owned chunk (momentum / second-moment state for that chunk only) and all-gather the result.
* Three phases so communication of later groups overlaps computation of earlier ones:
  launch every reduction -> per group wait / update / launch gather -> wait gathers and copy back.

This is the NCCL-decomposed baseline; ``archlab_b200.parallel.fused_zero`` replaces the reduce /
update / gather chain of the matrix groups with peer-memory kernels on NVLink.
"""
from __future__ import annotations

import torch
from torch import Tensor

from ..parallel import collectives as coll
from .muon import adamw_update, muon_update


class DistMuonAdamW(torch.optim.Optimizer):
    def __init__(self, param_groups: list[dict], group=None):
        super().__init__(param_groups, defaults={})
        self.pg = group
        self._optimizer_step = 0

    # ------------------------------------------------------------------ phase 1
    def _reduce_adamw(self, group: dict, infos: dict) -> None:
        ws = coll.world_size(self.pg)
        for p in group["params"]:
            if p.grad is None:
                continue
            grad = p.grad
            if p.numel() < 1024 or p.dim() == 0 or p.shape[0] % ws != 0:
                fut = coll.all_reduce_avg(grad, self.pg, async_op=True)
                infos[p] = dict(future=fut, grad_slice=grad, is_small=True)
            else:
                rows = p.shape[0] // ws
                gs = torch.empty((rows, *p.shape[1:]), dtype=grad.dtype, device=grad.device)
                fut = coll.reduce_scatter_avg(gs, grad, self.pg, async_op=True)
                infos[p] = dict(future=fut, grad_slice=gs, is_small=False)

    def _reduce_muon(self, group: dict, infos: dict, gi: int) -> None:
        params = group["params"]
        if not params:
            return
        ws = coll.world_size(self.pg)
        K = len(params)
        chunk = (K + ws - 1) // ws
        padded = chunk * ws
        p0 = params[0]
        stacked = torch.zeros(padded, *p0.shape, dtype=p0.grad.dtype, device=p0.device)
        torch._foreach_copy_(list(stacked[:K].unbind(0)), [p.grad for p in params])
        gchunk = torch.empty(chunk, *p0.shape, dtype=stacked.dtype, device=p0.device)
        fut = coll.reduce_scatter_avg(gchunk, stacked, self.pg, async_op=True)
        infos[gi] = dict(future=fut, grad_chunk=gchunk, stacked=stacked, chunk=chunk)

    # ------------------------------------------------------------------ phase 2
    def _compute_adamw(self, group: dict, infos: dict, gathers: list) -> None:
        ws, rk = coll.world_size(self.pg), coll.rank(self.pg)
        for p in group["params"]:
            if p not in infos:
                continue
            info = infos[p]
            info["future"].wait()
            gs = info["grad_slice"]
            if info["is_small"]:
                pslice = p.data
            else:
                rows = p.shape[0] // ws
                pslice = p.data[rk * rows:(rk + 1) * rows]
            st = self.state[p]
            if "exp_avg" not in st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(pslice)
                st["exp_avg_sq"] = torch.zeros_like(pslice)
            st["step"] += 1
            adamw_update(pslice, gs, st["exp_avg"], st["exp_avg_sq"], step=st["step"], lr=group["lr"],
                         beta1=group["betas"][0], beta2=group["betas"][1], eps=group["eps"],
                         wd=group["weight_decay"], cautious=bool(group.get("cautious_weight_decay", False)))
            if not info["is_small"]:
                fut = coll.all_gather_into(p.data, pslice.contiguous(), self.pg, async_op=True)
                gathers.append(dict(future=fut, params=None))

    def _compute_muon(self, group: dict, info: dict, gathers: list) -> None:
        params = group["params"]
        ws, rk = coll.world_size(self.pg), coll.rank(self.pg)
        info["future"].wait()
        K, chunk = len(params), info["chunk"]
        p0 = params[0]
        shape = p0.shape
        start = rk * chunk
        owned = max(0, min(chunk, K - start))
        st = self.state[p0]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros(chunk, *shape, dtype=p0.dtype, device=p0.device)
            sshape = (chunk, shape[-2], 1) if shape[-2] >= shape[-1] else (chunk, 1, shape[-1])
            st["second_momentum_buffer"] = torch.zeros(sshape, dtype=p0.dtype, device=p0.device)
        red_dim = -1 if shape[-2] >= shape[-1] else -2
        updated = torch.zeros(chunk, *shape, dtype=p0.dtype, device=p0.device)
        if owned > 0:
            torch._foreach_copy_(list(updated[:owned].unbind(0)), [p.data for p in params[start:start + owned]])
            muon_update(info["grad_chunk"][:owned], updated[:owned], st["momentum_buffer"][:owned],
                        st["second_momentum_buffer"][:owned], momentum=group["momentum"],
                        lr=group["lr"] * max(1.0, shape[-2] / shape[-1]) ** 0.5, wd=group["weight_decay"],
                        beta2=group["beta2"] if group["beta2"] is not None else 0.0,
                        ns_steps=group["ns_steps"], red_dim=red_dim,
                        hyperball=bool(group.get("hyperball", False)),
                        equilibrate_exponent=float(group.get("equilibrate_exponent", 0.0)))
        out = info["stacked"].to(p0.dtype) if info["stacked"].dtype != p0.dtype else info["stacked"]
        fut = coll.all_gather_into(out, updated, self.pg, async_op=True)
        gathers.append(dict(future=fut, params=params, stacked=out))

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self):
        infos: dict = {}
        for gi, group in enumerate(self.param_groups):
            if group["kind"] == "adamw":
                self._reduce_adamw(group, infos)
            elif group["kind"] == "muon":
                self._reduce_muon(group, infos, gi)
            else:
                raise ValueError(f"Unknown optimizer kind for the distributed driver: {group['kind']}")
        gathers: list = []
        for gi, group in enumerate(self.param_groups):
            if group["kind"] == "adamw":
                self._compute_adamw(group, infos, gathers)
            elif gi in infos:
                self._compute_muon(group, infos[gi], gathers)
        for g in gathers:
            g["future"].wait()
            if g["params"] is not None:
                params = g["params"]
                torch._foreach_copy_([p.data for p in params], list(g["stacked"][:len(params)].unbind(0)))
        self._optimizer_step += 1
