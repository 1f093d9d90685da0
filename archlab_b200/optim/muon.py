"""Muon + AdamW mixed optimizer (single process) and the math shared with the distributed driver.

Semantics follow the reference's ``MuonAdamW`` (src/archlab/optimizers/speedrun.py:31-231 fused
step functions, :239-439 optimizer, :758-842 grouping):

* ``adamw``: lerp moments, bias correction, decoupled (optionally cautious) weight decay;
* ``muon``: Nesterov momentum -> optional row/column equilibration -> Polar Express quintic
  Newton-Schulz (5 coefficient triples, bf16 when the compute dtype is bf16, tall/wide branches) ->
  NorMuon factored second-moment variance reduction -> cautious weight decay + update, or the MuonH
  Frobenius-hyperball projection; learning rate scaled by ``sqrt(max(1, rows/cols))``;
* ``adamh``: Adam direction projected back to each matrix's Frobenius sphere.

All same-shape Muon parameters are processed as one stacked ``(K, m, n)`` tensor.  On CUDA the
Newton-Schulz products run on the tcgen05 GEMM (``ops.gemm``) instead of cuBLAS ``bmm``.
"""
from __future__ import annotations

import torch
from torch import Tensor

POLAR_EXPRESS_COEFFS = [
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
]


def adamw_update(p: Tensor, grad: Tensor, exp_avg: Tensor, exp_avg_sq: Tensor, *, step: int, lr: float,
                 beta1: float, beta2: float, eps: float, wd: float, cautious: bool = False) -> None:
    exp_avg.lerp_(grad.to(exp_avg.dtype), 1 - beta1)
    exp_avg_sq.lerp_(grad.to(exp_avg_sq.dtype).square(), 1 - beta2)
    bias1 = 1 - beta1 ** step
    bias2 = 1 - beta2 ** step
    denom = (exp_avg_sq / bias2).sqrt() + eps
    update = exp_avg / denom
    if cautious:
        mask = (update * p) >= 0
        p.sub_(lr * wd * p * mask)
    else:
        p.mul_(1 - lr * wd)
    p.add_(update.to(p.dtype), alpha=-lr / bias1)


def _mm(a: Tensor, b: Tensor, *, b_mn: bool, a_mn: bool = False, aux: Tensor | None = None,
        alpha: float = 1.0, beta: float = 0.0) -> Tensor:
    """alpha * op(a) @ op(b) + beta * aux on stacked matrices (``ops.gemm`` operand convention);
    tcgen05 kernel on CUDA bf16."""
    if (a.is_cuda and a.dtype == torch.bfloat16 and a.size(-1) % 8 == 0 and b.size(-1) % 8 == 0
            and min(a.size(-1), a.size(-2), b.size(-1), b.size(-2)) >= 64):
        from ..ops.gemm import EPI_AXPBY, EPI_SCALE, gemm

        return gemm(a, b, a_mn=a_mn, b_mn=b_mn, aux=aux, epi=EPI_AXPBY if aux is not None else EPI_SCALE,
                    alpha=alpha, beta=beta)
    out = alpha * ((a.mT if a_mn else a) @ (b if b_mn else b.mT))
    if aux is not None:
        out = out + beta * aux
    return out


def polar_express(g: Tensor, ns_steps: int = 5, *, bf16: bool | None = None) -> Tensor:
    """Approximate zeroth power (orthogonalisation) of stacked matrices ``(K, m, n)``."""
    if bf16 is None:
        bf16 = g.is_cuda
    X = g.bfloat16() if bf16 else g
    X = X / (X.norm(dim=(-2, -1), keepdim=True) * 1.01 + 1e-6)
    X = X.contiguous()
    tall = g.size(-2) > g.size(-1)
    for a, b, c in POLAR_EXPRESS_COEFFS[:ns_steps]:
        if tall:
            # A = X^T X ; B = b A + c A A ; X = a X + X B          (A symmetric)
            A = _mm(X, X, a_mn=True, b_mn=True)
            B = _mm(A, A, b_mn=False, aux=A, alpha=c, beta=b)
            X = _mm(X, B, b_mn=False, aux=X, alpha=1.0, beta=a)
        else:
            A = _mm(X, X, b_mn=False)
            B = _mm(A, A, b_mn=False, aux=A, alpha=c, beta=b)
            X = _mm(B, X, b_mn=True, aux=X, alpha=1.0, beta=a)
    return X


def muon_update(stacked_grads: Tensor, stacked_params: Tensor, momentum_buffer: Tensor,
                second_momentum_buffer: Tensor, *, momentum: float, lr: float, wd: float, beta2: float,
                ns_steps: int, red_dim: int, hyperball: bool = False, equilibrate_exponent: float = 0.0,
                bf16: bool | None = None) -> None:
    momentum_buffer.lerp_(stacked_grads, 1 - momentum)
    g = stacked_grads.lerp_(momentum_buffer, momentum)
    if equilibrate_exponent != 0.0:
        g32 = g.float()
        row = g32.square().sum(dim=-1, keepdim=True)
        col = g32.square().sum(dim=-2, keepdim=True)
        row_scale = torch.where(row > 1e-16, row.pow(equilibrate_exponent), torch.ones_like(row))
        col_scale = torch.where(col > 1e-16, col.pow(equilibrate_exponent), torch.ones_like(col))
        g = (g32 * row_scale * col_scale).to(g.dtype)
    g = polar_express(g, ns_steps, bf16=bf16)
    # NorMuon variance reduction
    v_mean = g.float().square().mean(dim=red_dim, keepdim=True)
    red = g.size(red_dim)
    v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * red).sqrt()
    second_momentum_buffer.lerp_(v_mean.to(second_momentum_buffer.dtype), 1 - beta2)
    step_size = second_momentum_buffer.clamp_min(1e-10).rsqrt()
    scaled = (v_mean * red) * step_size.float().square()
    v_norm_new = scaled.sum(dim=(-2, -1), keepdim=True).sqrt()
    final_scale = step_size * (v_norm / v_norm_new.clamp_min(1e-10))
    g = g * final_scale.to(g.dtype)
    if hyperball:
        p32, d32 = stacked_params.float(), g.float()
        pn = p32.norm(dim=(-2, -1), keepdim=True)
        dn = d32.norm(dim=(-2, -1), keepdim=True).clamp_min(1e-10)
        upd = p32 - lr * d32 * (pn / dn)
        un = upd.norm(dim=(-2, -1), keepdim=True).clamp_min(1e-10)
        stacked_params.copy_((upd * (pn / un)).to(stacked_params.dtype))
    else:
        g = g.to(stacked_params.dtype)
        mask = (g * stacked_params) >= 0
        stacked_params.sub_(lr * g + lr * wd * stacked_params * mask)


def adamh_update(stacked_grads, stacked_params, exp_avg, exp_avg_sq, *, step, lr, beta1, beta2, eps):
    exp_avg.lerp_(stacked_grads, 1 - beta1)
    exp_avg_sq.lerp_(stacked_grads.square(), 1 - beta2)
    direction = (exp_avg / (1 - beta1 ** step)) / ((exp_avg_sq / (1 - beta2 ** step)).sqrt() + eps)
    p32, d32 = stacked_params.float(), direction.float()
    pn = p32.norm(dim=(-2, -1), keepdim=True)
    dn = d32.norm(dim=(-2, -1), keepdim=True).clamp_min(1e-10)
    upd = p32 - lr * d32 * (pn / dn)
    un = upd.norm(dim=(-2, -1), keepdim=True).clamp_min(1e-10)
    stacked_params.copy_((upd * (pn / un)).to(stacked_params.dtype))


class MuonAdamW(torch.optim.Optimizer):
    """Single-process mixed optimizer over groups of ``kind in {adamw, muon, adamh}``."""

    def __init__(self, param_groups: list[dict]):
        super().__init__(param_groups, defaults={})
        self._optimizer_step = 0

    def _step_adamw(self, group: dict) -> None:
        every = int(group.get("update_every", 1))
        should = self._optimizer_step % every == every - 1
        for p in group["params"]:
            if p.grad is None:
                continue
            st = self.state[p]
            grad = p.grad
            if every > 1:
                if "pending_grad" not in st:
                    st["pending_grad"] = torch.zeros_like(grad)
                st["pending_grad"].add_(grad)
                if not should:
                    continue
                grad = st["pending_grad"]
            if "exp_avg" not in st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(p)
                st["exp_avg_sq"] = torch.zeros_like(p)
            st["step"] += 1
            adamw_update(p.data, grad, st["exp_avg"], st["exp_avg_sq"], step=st["step"], lr=group["lr"],
                         beta1=group["betas"][0], beta2=group["betas"][1], eps=group["eps"],
                         wd=group["weight_decay"], cautious=bool(group.get("cautious_weight_decay", False)))
            if every > 1:
                st["pending_grad"].zero_()

    def _step_adamh(self, group: dict) -> None:
        params = list(group["params"])
        if not params:
            return
        if any(p.grad is None for p in params):
            raise RuntimeError("AdamH requires a gradient for every grouped matrix")
        st = self.state[params[0]]
        if "exp_avg" not in st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros(len(params), *params[0].shape, dtype=params[0].dtype,
                                        device=params[0].device)
            st["exp_avg_sq"] = torch.zeros_like(st["exp_avg"])
        st["step"] += 1
        sp = torch.stack([p.data for p in params])
        adamh_update(torch.stack([p.grad for p in params]), sp, st["exp_avg"], st["exp_avg_sq"],
                     step=st["step"], lr=group["lr"], beta1=group["betas"][0], beta2=group["betas"][1],
                     eps=group["eps"])
        torch._foreach_copy_([p.data for p in params], list(sp.unbind(0)))

    def _step_muon(self, group: dict) -> None:
        params: list[Tensor] = group["params"]
        if not params:
            return
        p0 = params[0]
        st = self.state[p0]
        K, shape = len(params), p0.shape
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros(K, *shape, dtype=p0.dtype, device=p0.device)
            sshape = (K, shape[-2], 1) if shape[-2] >= shape[-1] else (K, 1, shape[-1])
            st["second_momentum_buffer"] = torch.zeros(sshape, dtype=p0.dtype, device=p0.device)
        red_dim = -1 if shape[-2] >= shape[-1] else -2
        sg = torch.stack([p.grad for p in params])
        sp = torch.stack([p.data for p in params])
        muon_update(sg, sp, st["momentum_buffer"], st["second_momentum_buffer"], momentum=group["momentum"],
                    lr=group["lr"] * max(1.0, shape[-2] / shape[-1]) ** 0.5, wd=group["weight_decay"],
                    beta2=group["beta2"] if group["beta2"] is not None else 0.0, ns_steps=group["ns_steps"],
                    red_dim=red_dim, hyperball=bool(group.get("hyperball", False)),
                    equilibrate_exponent=float(group.get("equilibrate_exponent", 0.0)))
        torch._foreach_copy_([p.data for p in params], list(sp.unbind(0)))

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            kind = group["kind"]
            if kind == "adamw":
                self._step_adamw(group)
            elif kind == "muon":
                self._step_muon(group)
            elif kind == "adamh":
                self._step_adamh(group)
            else:
                raise ValueError(f"Unknown optimizer kind: {kind}")
        self._optimizer_step += 1
