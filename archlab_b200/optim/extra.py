"""Optimizers beyond the speedrun Muon / AdamW pair.

* ``HeadwiseMuon``: heavy-ball momentum, rows split into independent per-head matrices, 8 fast + 2
  stabilising Newton-Schulz steps in fp32, update scaled to a target RMS
  (src/archlab/optimizers/headwise_muon.py:16-76).
* ``Muown``: weight-normalised Muon: each row is ``g * v / |v|``; the row gain ``g`` follows Adam, the
  direction ``v`` gets the orthogonalised (tangent) gradient; tensor-parallel shards are gathered
  before orthogonalisation; optional fp16 momentum with a power-of-two scale
  (src/archlab/optimizers/muown.py:13-129).
* ``ShardedAdafactor``: factored second moments (epsilon inside the statistic), relative step size,
  RMS clipping, row-chunked temporaries, optional row-owner process group, stochastic bf16 stores
  (src/archlab/optimizers/sharded_adafactor.py:33-252).
* ``sinkhorn_direction`` / ``SinkhornTables``: DeepSeek-V4.1 table optimizer: Nesterov momentum, row
  threshold, K alternating row / column L2 normalisations kept as two scale vectors, ``sqrt(cols)``
  and a 0.18 correction (src/archlab/optimizers/sinkhorn.py:17-168).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops.quant import stochastic_bfloat16

_FAST = (3.4445, -4.775, 2.0315)
_STABLE = (2.0, -1.5, 0.5)


def orthogonalized_direction(gradient: torch.Tensor, fast_steps: int = 8, stable_steps: int = 2) -> torch.Tensor:
    """Batched fp32 Newton-Schulz on ``[..., m, n]``; an exactly zero matrix stays zero."""
    if gradient.ndim < 2 or gradient.dtype != torch.float32:
        raise ValueError("complete FP32 matrices are required")
    tall = gradient.shape[-2] > gradient.shape[-1]
    x = gradient.mT if tall else gradient
    nrm = x.norm(dim=(-2, -1), keepdim=True)
    x = x / torch.where(nrm > 0, nrm, torch.ones_like(nrm))
    for a, b, c in [_FAST] * fast_steps + [_STABLE] * stable_steps:
        xx = x @ x.mT
        x = a * x + (b * xx + c * (xx @ xx)) @ x
    return x.mT if tall else x


class HeadwiseMuon(torch.optim.Optimizer):
    """A group's ``head_dim`` cuts the rows into consecutive blocks orthogonalised independently."""

    def __init__(self, params, lr=1e-5, momentum=0.95, weight_decay=0.1, update_rms=0.18):
        vals = (lr, momentum, weight_decay, update_rms)
        if any(not math.isfinite(v) for v in vals) or lr < 0 or not 0 <= momentum < 1 or weight_decay < 0 or update_rms <= 0:
            raise ValueError("invalid Muon hyperparameters")
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, update_rms=update_rms, head_dim=None))
        seen = set()
        for g in self.param_groups:
            hd = g["head_dim"]
            for p in g["params"]:
                if id(p) in seen or p.ndim != 2 or p.dtype != torch.float32 or not p.requires_grad:
                    raise ValueError("unique trainable complete FP32 matrix parameters are required")
                if hasattr(p, "to_local"):
                    raise ValueError("orthogonalizing distributed shards is not supported")
                if hd is not None and (type(hd) is not int or hd < 1 or p.shape[0] % hd):
                    raise ValueError("head_dim must divide matrix rows")
                seen.add(id(p))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse or p.grad.dtype != torch.float32:
                    raise ValueError("dense globally reduced FP32 gradients are required")
                st = self.state[p]
                if not st:
                    st["momentum_buffer"] = torch.zeros_like(p)
                m = st["momentum_buffer"].mul_(g["momentum"]).add_(p.grad)
                d = p.grad + g["momentum"] * m
                mats = d if g["head_dim"] is None else d.unflatten(0, (-1, g["head_dim"]))
                upd = orthogonalized_direction(mats)
                scale = g["update_rms"] * math.sqrt(max(mats.shape[-2:]))
                p.mul_(1 - g["lr"] * g["weight_decay"]).add_(upd.reshape_as(p), alpha=-g["lr"] * scale)
        return loss


def _ns_bf16(matrix: torch.Tensor, steps: int, dtype=torch.bfloat16) -> torch.Tensor:
    x = matrix.to(dtype)
    tall = x.shape[0] > x.shape[1]
    if tall:
        x = x.T
    x = x / (x.norm() + 1e-7)
    for _ in range(steps):
        a = x @ x.T
        b = torch.addmm(a, a, a, beta=_FAST[1], alpha=_FAST[2])
        x = torch.addmm(x, b, x, beta=_FAST[0])
    return (x.T if tall else x).float()


class Muown(torch.optim.Optimizer):
    def __init__(self, params, lr=3e-6, momentum=0.95, betas=(0.95, 0.95), eps=1e-8, ns_steps=10, update_scale=0.5,
                 tp_group=None, momentum_dtype=None, orthogonalization_dtype=torch.bfloat16):
        super().__init__(params, dict(lr=lr, momentum=momentum, betas=betas, eps=eps, ns_steps=ns_steps, update_scale=update_scale))
        self.tp_group, self.momentum_dtype, self.ns_dtype = tp_group, momentum_dtype, orthogonalization_dtype

    def _shard(self, p):
        axis = getattr(p, "partition_dim", -1)
        if not getattr(p, "tensor_model_parallel", False) or axis < 0 or self.tp_group is None:
            return None, -1
        return self.tp_group, axis

    def _row_sum(self, p, value):
        out = value.sum(1, keepdim=True)
        group, axis = self._shard(p)
        if axis == 1 and dist.get_world_size(group) > 1:
            dist.all_reduce(out, group=group)
        return out

    def _orthogonalize(self, p, direction, steps):
        group, axis = self._shard(p)
        size = dist.get_world_size(group) if group is not None else 1
        if size == 1:
            return _ns_bf16(direction, steps, self.ns_dtype), direction.shape
        parts = [torch.empty_like(direction) for _ in range(size)]
        dist.all_gather(parts, direction.contiguous(), group=group)
        full = torch.cat(parts, dim=axis)
        res = _ns_bf16(full, steps, self.ns_dtype)
        return res.chunk(size, dim=axis)[dist.get_rank(group)], full.shape

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for grp in self.param_groups:
            b1, b2 = grp["betas"]
            for p in grp["params"]:
                if p.grad is None:
                    continue
                s = self.state[p]
                if not s:
                    if p.ndim != 2:
                        raise ValueError("Muown matrix groups must contain two-dimensional weights")
                    nrm = self._row_sum(p, p.float().square()).sqrt()
                    s.update(step=0, g=nrm.clone(), v_norm=nrm.clamp_min(1e-12), m_g=torch.zeros_like(nrm), v_g=torch.zeros_like(nrm),
                             momentum_buffer=torch.zeros_like(p, dtype=self.momentum_dtype or p.dtype))
                    if self.momentum_dtype == torch.float16:
                        s["momentum_scale"] = torch.ones((), device=p.device)
                s["step"] += 1
                g, vn = s["g"], s["v_norm"]
                grad = p.grad.float()
                u = p.float() / g.abs().clamp_min(1e-12) * g.sign().masked_fill(g == 0, 1)
                gn = self._row_sum(p, grad.square()).sqrt().clamp_min(1e-12)
                u = torch.where(g == 0, grad / gn, u)                 # zero rows take their first direction from the gradient
                v = u * vn
                grad_g = self._row_sum(p, grad * u)
                grad_v = (g / vn) * (grad - u * grad_g)               # tangent component
                mom = s["momentum_buffer"].float()
                if "momentum_scale" in s:
                    mom.mul_(s["momentum_scale"])
                mom.mul_(grp["momentum"]).add_(grad_v)
                if "momentum_scale" in s:
                    sc = torch.exp2(torch.ceil(torch.log2(mom.abs().amax().clamp_min(2.0 ** -110))))
                    s["momentum_buffer"].copy_(mom / sc)
                    s["momentum_scale"].copy_(sc)
                else:
                    s["momentum_buffer"].copy_(mom)
                upd, shape = self._orthogonalize(p, grad_v.add(mom, alpha=grp["momentum"]), grp["ns_steps"])
                v.add_(upd, alpha=-grp["lr"] * 0.2 * math.sqrt(max(shape)) * grp["update_scale"])
                s["m_g"].lerp_(grad_g, 1 - b1)
                s["v_g"].lerp_(grad_g.square(), 1 - b2)
                den = (s["v_g"] / (1 - b2 ** s["step"])).sqrt().add_(grp["eps"])
                g.addcdiv_(s["m_g"], den, value=-grp["lr"] / (1 - b1 ** s["step"]))
                vn.copy_(self._row_sum(p, v.square()).sqrt().clamp_min(1e-12))
                p.copy_(g * (v / vn))
        return loss


class ShardedAdafactor(torch.optim.Optimizer):
    """Parameters are 1-D, 2-D ``[rows, cols]`` or 3-D ``[batch, rows, cols]`` LOCAL row shards; a
    parameter attribute ``row_group`` (process group) and ``global_rows`` describe the sharding."""

    def __init__(self, params, lr=1e-4, *, eps=1e-30, parameter_floor=1e-3, beta2_decay=-0.8, clip_threshold=1.0,
                 chunk_elements=16 * 1024 * 1024, stochastic_rounding=True, weight_decay=0.0):
        if not 0 < lr <= 1 or eps <= 0 or not -1 <= beta2_decay < 0:
            raise ValueError("invalid Adafactor hyperparameters")
        if not math.isfinite(weight_decay) or weight_decay < 0:
            raise ValueError("matrix weight decay must be finite and nonnegative")
        super().__init__(params, dict(lr=lr, eps=eps, parameter_floor=parameter_floor, beta2_decay=beta2_decay,
                                     clip_threshold=clip_threshold, chunk_elements=chunk_elements,
                                     stochastic_rounding=stochastic_rounding, weight_decay=weight_decay))
        self.last_metrics: dict = {}

    @staticmethod
    def _sum(t, group):
        if group is not None and dist.get_world_size(group) > 1:
            dist.all_reduce(t, group=group)
        return t

    @staticmethod
    def _store(dst, candidate, stochastic):
        res = stochastic_bfloat16(candidate) if dst.dtype == torch.bfloat16 and stochastic else candidate.to(dst.dtype)
        changed = (res != dst).sum()
        dst.copy_(res)
        return changed

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        changed, updated = 0, 0
        for o in self.param_groups:
            for p in o["params"]:
                if p.grad is None:
                    continue
                if p.ndim not in (1, 2, 3) or p.grad.is_sparse or p.grad.shape != p.shape:
                    raise ValueError("expected dense gradients with the local parameter shape")
                group = getattr(p, "row_group", None)
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    if p.ndim > 1:
                        st["row"] = torch.zeros((*p.shape[:-1], 1), device=p.device)
                        st["col"] = torch.zeros((*p.shape[:-2], 1, p.shape[-1]), device=p.device)
                    else:
                        st["variance"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                mix, rho, eps = st["step"] ** o["beta2_decay"], min(o["lr"], st["step"] ** -0.5), o["eps"]
                if p.ndim == 1:
                    g = p.grad.float()
                    st["variance"].lerp_(g.square().add_(eps), mix)
                    upd = g * st["variance"].rsqrt()
                    sq = self._sum(torch.stack([p.float().square().sum(), upd.square().sum(), g.new_tensor(float(p.numel()))]), group)
                    alpha = rho * max(o["parameter_floor"], math.sqrt(float(sq[0] / sq[2])))
                    alpha /= max(1.0, math.sqrt(float(sq[1] / sq[2])) / o["clip_threshold"])
                    changed += int(self._store(p, p.float().add_(upd, alpha=-alpha), o["stochastic_rounding"]))
                else:
                    cols, rows = p.shape[-1], p.shape[-2]
                    B = 1 if p.ndim == 2 else p.shape[0]
                    v, g = p.view(B, rows, cols), p.grad.view(B, rows, cols)
                    row, col = st["row"].view(B, rows, 1), st["col"].view(B, 1, cols)
                    chunk = max(1, o["chunk_elements"] // cols)
                    global_rows = int(getattr(p, "global_rows", rows))
                    col_sum = torch.zeros_like(col)
                    psq = torch.zeros(B, 1, 1, device=p.device)
                    for r0 in range(0, rows, chunk):
                        sq = g[:, r0:r0 + chunk].float().square().add_(eps)
                        row[:, r0:r0 + chunk].lerp_(sq.mean(-1, keepdim=True), mix)
                        col_sum += sq.sum(-2, keepdim=True)
                        psq += v[:, r0:r0 + chunk].float().square().sum((-2, -1), keepdim=True)
                    row_mean = row.sum(-2, keepdim=True)
                    for t in (col_sum, psq, row_mean):
                        self._sum(t, group)
                    col.lerp_(col_sum / global_rows, mix)
                    row_mean.div_(global_rows).clamp_min_(eps)
                    scale = (psq / (global_rows * cols)).sqrt_().clamp_min_(o["parameter_floor"]).mul_(rho)
                    inv = lambda r0: (row[:, r0:r0 + chunk] / row_mean * col).clamp_min_(eps).rsqrt_()
                    usq = torch.zeros_like(psq)
                    for r0 in range(0, rows, chunk):
                        usq += inv(r0).mul_(g[:, r0:r0 + chunk]).square().sum((-2, -1), keepdim=True)
                    self._sum(usq, group)
                    scale.div_((usq / (global_rows * cols)).sqrt_().div_(o["clip_threshold"]).clamp_min_(1))
                    for r0 in range(0, rows, chunk):
                        old = v[:, r0:r0 + chunk]
                        cand = old.float() - inv(r0).mul_(g[:, r0:r0 + chunk]).mul_(scale)
                        if o["weight_decay"]:
                            cand.add_(old.float(), alpha=-rho * o["weight_decay"])
                        changed += int(self._store(old, cand, o["stochastic_rounding"]))
                updated += 1
        self.last_metrics = {"updated_parameter_tensors": updated, "changed_local_elements": changed}
        return loss


def sinkhorn_direction(update: torch.Tensor, *, global_rows=None, group=None, steps: int = 11, tau: float = 1e-3,
                       eps: float = 1e-20) -> torch.Tensor:
    """RMS-normalised direction of a (row-sharded) table update; a zero update stays exactly zero."""
    if update.ndim != 2 or steps < 1 or steps % 2 != 1:
        raise ValueError("Sinkhorn requires a matrix and a positive odd iteration count")
    if tau < 0 or eps <= 0 or (global_rows is not None and global_rows < 1):
        raise ValueError("invalid Sinkhorn threshold, epsilon or row count")
    sq = update.float().square()
    rho = sq.sum(-1).sqrt()
    total = rho.sum()
    if group is not None:
        dist.all_reduce(total, group=group)
    rows = update.shape[0] if global_rows is None else global_rows
    row = (rho > tau * total / rows).float()
    col = torch.ones(update.shape[1], device=update.device)
    for it in range(steps):
        if it % 2 == 0:
            n = (sq @ col.square()).sqrt() * row
            row = torch.where(n > 0, row / (n + eps), torch.zeros_like(row))
        else:
            part = sq.T @ row.square()
            if group is not None:
                dist.all_reduce(part, group=group)
            n = part.sqrt() * col
            col = torch.where(n > 0, col / (n + eps), torch.zeros_like(col))
    return update.float() * row[:, None] * col[None, :] * math.sqrt(update.shape[1])


class SinkhornTables(torch.optim.Optimizer):
    """Hashed-embedding tables: fp32 Nesterov momentum (the only full-size state), Sinkhorn direction,
    correction 0.18, no weight decay, stochastic bf16 stores."""

    def __init__(self, params, lr=5e-4, beta=0.95, correction=0.18, steps=11, tau=1e-3, stochastic_rounding=True):
        super().__init__(params, dict(lr=lr, beta=beta, correction=correction, steps=steps, tau=tau,
                                     stochastic_rounding=stochastic_rounding))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for o in self.param_groups:
            for p in o["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st.update(step=0, momentum=torch.zeros_like(p, dtype=torch.float32))
                g = p.grad.float()
                m = st["momentum"].mul_(o["beta"]).add_(g, alpha=1 - o["beta"])
                upd = m.mul(o["beta"]).add_(g, alpha=1 - o["beta"])
                d = sinkhorn_direction(upd, global_rows=getattr(p, "global_rows", None), group=getattr(p, "row_group", None),
                                       steps=o["steps"], tau=o["tau"])
                cand = p.float() - o["correction"] * o["lr"] * d
                p.copy_(stochastic_bfloat16(cand) if p.dtype == torch.bfloat16 and o["stochastic_rounding"] else cand.to(p.dtype))
                st["step"] += 1
        return loss
