"""Layer-wise distributed Muon with logical matrix splits, for the mesh trainer.

What the reference gets from Megatron's layer-wise distributed Muon plus its Qwen3.8 adapter
(src/archlab/megatron/qwen38_muon.py:120-264, placement :148-153 of its own notes):

* a fused physical parameter is orthogonalised as several *logical* matrices: a tensor tagged
  ``archlab_muon_split_rows = r`` of shape ``[R, C]`` is the stack ``[R / r, r, C]`` (attention Q per head, GDN q/k/v
  per head, expert gate / up halves); stacked expert tensors ``[E, R, C]`` contribute ``E x R / r`` matrices;
* Nesterov momentum 0.95, eight Polar-Express Newton-Schulz steps on Frobenius-normalised matrices in bf16,
  update scale ``0.2 sqrt(max(r, C))`` per logical matrix, decoupled weight decay;
* whole parameters are dealt to the ranks of the data group by longest-processing-time-first, the owner keeps the
  momentum and computes the update, everybody receives the new weights.

Here the Newton-Schulz products run on the batched tcgen05 GEMM (``optim.muon._mm``) on a GPU; gradients are
averaged with one all-reduce over a flat view per owner and the new weights travel in one broadcast per owner.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..parallel import collectives as coll
from .muon import _mm

# Eight-step Polar Express schedule (published coefficients; the last triple repeats the classical cubic)
POLAR_EXPRESS_8 = ((8.2051, -22.9019, 16.4607), (4.0664, -2.8612, 0.5184), (3.9096, -2.8234, 0.5250), (3.2856, -2.4153, 0.4853),
                   (2.2779, -1.6198, 0.3985), (1.8726, -1.2307, 0.3585), (1.8564, -1.2132, 0.3568), (1.8750, -1.2500, 0.3750))
FROBENIUS_EPS = 1e-14


def muon_recipe() -> dict:
    """The recipe as recorded next to a run (what must not drift between attempts)."""
    return {"momentum": 0.95, "nesterov": True, "coefficient_schedule": "polar_express", "newton_schulz_steps": len(POLAR_EXPRESS_8),
            "frobenius_normalization_epsilon": FROBENIUS_EPS, "scale": "0.2 * sqrt(max(rows, columns)) per logical matrix",
            "matmul": "bf16 Newton-Schulz products, fp32 accumulation",
            "fused_parameter_splitting": {"attention_q": "per head", "gdn_qkv": "per q/k/v head", "expert_fc1": "gate/up halves"},
            "placement": "longest-processing-time whole-parameter placement over the data group"}


def logical_matrices(t: torch.Tensor, split_rows: int | None) -> torch.Tensor:
    """View of a physical parameter (or gradient) as ``[count, rows, cols]`` logical matrices."""
    if t.ndim not in (2, 3):
        raise ValueError("Muon takes 2-D matrices or stacks of them")
    rows_total, cols = t.shape[-2], t.shape[-1]
    rows = int(split_rows) if split_rows else rows_total
    if rows_total % rows:
        raise ValueError(f"cannot split {tuple(t.shape)} into {rows}-row matrices")
    return t.reshape(-1, rows, cols)


def orthogonalize(matrices: torch.Tensor, *, bf16: bool = True) -> torch.Tensor:
    """Approximate polar factor of every matrix of the stack (fp32 in, fp32 out)."""
    if matrices.ndim != 3:
        raise ValueError("expected [count, rows, cols]")
    wide = matrices.size(-2) <= matrices.size(-1)
    x = matrices if wide else matrices.mT                      # work on the orientation with the small Gram matrix
    x = x / x.square().sum(dim=(-2, -1), keepdim=True).sqrt().clamp_min(FROBENIUS_EPS)
    x = (x.to(torch.bfloat16) if bf16 else x).contiguous()
    for a, b, c in POLAR_EXPRESS_8:
        gram = _mm(x, x, b_mn=False)                           # X X^T
        poly = _mm(gram, gram, b_mn=False, aux=gram, alpha=c, beta=b)      # c G G + b G   (G symmetric)
        x = _mm(poly, x, b_mn=True, aux=x, alpha=1.0, beta=a)  # (b G + c G^2) X + a X
    x = x.float()
    return x if wide else x.mT


def lpt_placement(costs: list[float], world: int) -> list[int]:
    """Owner of every item: items in descending cost, each to the currently least-loaded rank (ties: lowest rank)."""
    load = [0.0] * world
    owner = [0] * len(costs)
    for i in sorted(range(len(costs)), key=lambda i: (-costs[i], i)):
        r = min(range(world), key=lambda r: (load[r], r))
        owner[i] = r
        load[r] += costs[i]
    return owner


@dataclass
class _Entry:
    name: str
    param: torch.nn.Parameter
    split_rows: int | None
    owner: int
    momentum: torch.Tensor | None = None      # fp32, owner only
    master: torch.Tensor | None = None        # fp32 master weights, owner only (the model may be bf16)


class SplitRowsMuon:
    """Muon over the parameters tagged ``archlab_optimizer == "muon"``; everything else belongs to another optimizer."""

    def __init__(self, named_params, *, lr: float = 0.02, weight_decay: float = 0.0, momentum: float = 0.95,
                 extra_scale: float = 0.2, group=None, bf16: bool | None = None, average: bool = True):
        named = [(n, p) for n, p in named_params if p.requires_grad and getattr(p, "archlab_optimizer", None) == "muon"]
        if not named:
            raise ValueError("no parameter is tagged for Muon")
        self.group = group
        self.world, self.rank = coll.world_size(group), coll.rank(group)
        self.lr, self.wd, self.mu, self.extra = lr, weight_decay, momentum, extra_scale
        costs = []
        for _, p in named:
            lm = logical_matrices(p, getattr(p, "archlab_muon_split_rows", None))
            k, r, c = lm.shape
            costs.append(float(k) * r * c * min(r, c))          # Newton-Schulz work of the parameter
        owners = lpt_placement(costs, self.world)
        self.entries = [_Entry(n, p, getattr(p, "archlab_muon_split_rows", None), o) for (n, p), o in zip(named, owners)]
        self.bf16, self.average = bf16, average       # average=False: gradients are summed and the caller scales them
        self.t = 0
        for e in self.entries:
            if e.owner == self.rank:
                e.momentum = torch.zeros_like(e.param, dtype=torch.float32)
                e.master = e.param.detach().float().clone()

    @property
    def params(self):
        return [e.param for e in self.entries]

    def placement(self) -> dict[str, int]:
        return {e.name: e.owner for e in self.entries}

    def state_bytes(self) -> int:
        return sum(e.momentum.numel() * 8 for e in self.entries if e.momentum is not None)

    def grad_sq_norm(self) -> torch.Tensor:
        """Sum of squares of the (already averaged) gradients, for clipping together with the other optimizer."""
        dev = self.entries[0].param.device
        sq = [e.param.grad.float().square().sum() for e in self.entries if e.param.grad is not None]
        return torch.stack(sq).sum() if sq else torch.zeros((), device=dev)

    @torch.no_grad()
    def reduce_gradients(self) -> None:
        """Mean (or sum) over the data group; one flat all-reduce per owner keeps the collective count at ``world``."""
        if self.world == 1:
            return
        for owner in range(self.world):
            mine = [e for e in self.entries if e.owner == owner and e.param.grad is not None]
            if not mine:
                continue
            flat = torch.cat([e.param.grad.reshape(-1).float() for e in mine])
            dist.all_reduce(flat, group=self.group)
            if self.average:
                flat.div_(self.world)
            off = 0
            for e in mine:
                n = e.param.numel()
                e.param.grad.copy_(flat[off:off + n].view_as(e.param.grad))
                off += n

    @torch.no_grad()
    def step(self, *, lr_scale: float = 1.0, grad_scale: float = 1.0) -> None:
        self.t += 1
        lr = self.lr * lr_scale
        for e in self.entries:
            if e.owner != self.rank:
                continue
            g = (e.param.grad if e.param.grad is not None else torch.zeros_like(e.param)).float()
            if grad_scale != 1.0:
                g = g * grad_scale
            e.momentum.mul_(self.mu).add_(g)
            direction = g.add(e.momentum, alpha=self.mu)                            # Nesterov look-ahead
            lm = logical_matrices(direction, e.split_rows)
            use_bf16 = direction.is_cuda if self.bf16 is None else self.bf16
            update = orthogonalize(lm, bf16=use_bf16) * (self.extra * math.sqrt(max(lm.size(-2), lm.size(-1))))
            if self.wd:
                e.master.mul_(1.0 - lr * self.wd)
            e.master.add_(update.view_as(e.master), alpha=-lr)
            e.param.copy_(e.master)
        if self.world > 1:
            for owner in range(self.world):
                mine = [e for e in self.entries if e.owner == owner]
                if not mine:
                    continue
                flat = torch.cat([e.param.detach().reshape(-1) for e in mine])
                dist.broadcast(flat, src=dist.get_global_rank(self.group, owner) if self.group is not None else owner,
                               group=self.group)
                off = 0
                for e in mine:
                    n = e.param.numel()
                    e.param.copy_(flat[off:off + n].view_as(e.param))
                    off += n
        for e in self.entries:
            e.param.grad = None

    def state_dict(self) -> dict:
        return {"t": self.t, "rank": self.rank, "world": self.world, "placement": self.placement(),
                "momentum": {e.name: e.momentum for e in self.entries if e.momentum is not None},
                "master": {e.name: e.master for e in self.entries if e.master is not None}}

    def load_state_dict(self, sd: dict) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank or sd["placement"] != self.placement():
            raise ValueError("Muon state belongs to another rank layout or parameter placement")
        self.t = int(sd["t"])
        for e in self.entries:
            if e.momentum is not None:
                e.momentum.copy_(sd["momentum"][e.name])
                e.master.copy_(sd["master"][e.name])
