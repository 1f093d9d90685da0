"""Mixture-of-experts building blocks: routers, grouped SwiGLU experts, expert parallelism.

* ``route``: score function in {softmax, sigmoid, sqrt_softplus} + aux-free selection bias + top-k;
  weights are renormalised over the selected experts and scaled
  (src/archlab/architectures/deepseek_v41_inference_moe.py:9-16, qwen38_flash_next.py:653-718).
* ``swiglu_clamped``: SiLU(gate clamp max) * up clamp(+-limit), optionally probability-weighted
  (deepseek_v41_swiglu.py:64-87, deepseek_v41_inference_moe.py:19-29).
* ``GroupedExperts``: stacked expert weights; tokens are sorted by expert and processed per
  contiguous segment (the permute + grouped-GEMM form the sm_100a MoE kernels implement).
* ``SparseMoE``: router + routed experts + shared expert(s) + Switch aux loss / z-loss statistics.
* ``ExpertParallelMoE``: counts all-to-all -> dispatch tokens + weights -> local experts -> return
  -> FP32 sum in ascending expert-id order (deterministic)
  (src/archlab/automodel/deepseek_v41_parallel.py:16-111).  Works over NCCL and gloo.
* ``balance_routers``: world-aggregated expert load -> sign or clipped-proportional bias update
  with CV / dead-expert metrics over a 20-step window (src/archlab/optimizers/router_balance.py:16-78).
"""
from __future__ import annotations

from collections import deque

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def route(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, *, top_k: int, score: str = "sqrt_softplus",
          route_scale: float = 1.0, renormalize: bool = True):
    """x [N, C], weight [E, C] -> (weights [N, k] fp32, indices [N, k], scores [N, E] fp32)."""
    logits = F.linear(x.float(), weight.float())
    if score == "softmax":
        scores = logits.softmax(-1)
    elif score == "sigmoid":
        scores = logits.sigmoid()
    elif score == "sqrt_softplus":
        scores = F.softplus(logits).sqrt()
    else:
        raise ValueError(f"unknown router score {score!r}")
    sel = scores if bias is None else scores + bias.float()
    idx = sel.topk(top_k, dim=-1).indices
    w = scores.gather(1, idx)
    if renormalize and top_k > 1:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * route_scale, idx, scores


def swiglu_clamped(gate: torch.Tensor, up: torch.Tensor, limit: float | None = None,
                   probability: torch.Tensor | None = None) -> torch.Tensor:
    g, u = gate.float(), up.float()
    if limit is not None:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    a = F.silu(g) * u
    if probability is not None:
        a = a * probability.float()
    return a


class GroupedExperts(nn.Module):
    """E experts with weights ``gate_up [E, 2I, C]`` and ``down [E, C, I]``."""

    def __init__(self, n_experts: int, dim: int, inter: int, *, swiglu_limit: float | None = None):
        super().__init__()
        self.n_experts, self.dim, self.inter, self.limit = n_experts, dim, inter, swiglu_limit
        self.gate_up = nn.Parameter(torch.empty(n_experts, 2 * inter, dim))
        self.down = nn.Parameter(torch.empty(n_experts, dim, inter))

    @torch.no_grad()
    def init_weights(self, std: float = 0.02):
        nn.init.normal_(self.gate_up, std=std)
        nn.init.normal_(self.down, std=std)

    def forward(self, x: torch.Tensor, expert_ids: torch.Tensor, probability: torch.Tensor | None = None,
                first_expert: int = 0) -> torch.Tensor:
        """x [M, C] rows, expert_ids [M] (global ids of experts owned here); returns [M, C] in fp32.
        Rows are processed in segments of equal expert id (stable sort = the dispatch permutation)."""
        order = expert_ids.argsort(stable=True)
        xs = x[order]
        ids = expert_ids[order] - first_expert
        counts = torch.bincount(ids, minlength=self.n_experts)
        out = xs.new_zeros(xs.shape, dtype=torch.float32)
        ps = None if probability is None else probability[order]
        start = 0
        for e, n in enumerate(counts.tolist()):
            if n == 0:
                continue
            seg = slice(start, start + n)
            h = F.linear(xs[seg], self.gate_up[e].to(xs.dtype))
            a = swiglu_clamped(h[:, : self.inter], h[:, self.inter:], self.limit, None if ps is None else ps[seg])
            out[seg] = F.linear(a.to(xs.dtype), self.down[e].to(xs.dtype)).float()
            start += n
        res = torch.empty_like(out)
        res[order] = out
        return res


def dense_linear(x: torch.Tensor, weight: torch.Tensor, fp8: bool = False) -> torch.Tensor:
    """Bias-free linear of the MoE blocks: on a GPU in bf16 the tcgen05 kernels (block-scaled FP8 forward when ``fp8``
    and the reduction width is a multiple of 128), otherwise ``F.linear``."""
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.size(1) % 8 == 0 and weight.size(0) % 8 == 0:
        from ..ops import blockscaled, native_linear

        if fp8 and blockscaled.block_fp8_supported(x, weight):
            return blockscaled.block_fp8_linear(x, weight)
        return native_linear.native_linear(x, weight)
    return F.linear(x, weight.to(x.dtype))


class SwiGLU(nn.Module):
    def __init__(self, dim: int, inter: int, limit: float | None = None, fp8: bool = False):
        super().__init__()
        self.gate_up = nn.Linear(dim, 2 * inter, bias=False)
        self.down = nn.Linear(inter, dim, bias=False)
        self.inter, self.limit, self.fp8 = inter, limit, fp8

    def forward(self, x):
        h = dense_linear(x, self.gate_up.weight, self.fp8)
        if h.is_cuda and h.dtype == torch.bfloat16:
            from ..ops import block_ops

            a = block_ops.swiglu(h.reshape(-1, h.size(-1)), self.limit).reshape(*h.shape[:-1], self.inter)
        else:
            a = swiglu_clamped(h[..., : self.inter], h[..., self.inter:], self.limit).to(x.dtype)
        return dense_linear(a, self.down.weight, self.fp8)


class SparseMoE(nn.Module):
    def __init__(self, dim: int, inter: int, n_experts: int, top_k: int, *, n_shared: int = 1, shared_inter: int | None = None,
                 score: str = "sqrt_softplus", route_scale: float = 1.0, swiglu_limit: float | None = None,
                 aux_free_bias: bool = True, gated_shared: bool = False):
        super().__init__()
        self.dim, self.n_experts, self.top_k, self.score, self.route_scale = dim, n_experts, top_k, score, route_scale
        self.router = nn.Parameter(torch.empty(n_experts, dim))
        self.register_buffer("e_score_correction_bias", torch.zeros(n_experts, dtype=torch.float32) if aux_free_bias else None)
        self.experts = GroupedExperts(n_experts, dim, inter, swiglu_limit=swiglu_limit)
        self.shared = SwiGLU(dim, (shared_inter or inter) * n_shared, swiglu_limit) if n_shared else None
        self.shared_gate = nn.Linear(dim, 1, bias=False) if (gated_shared and n_shared) else None
        self._cumulative_expert_load = None
        self.last_metrics: dict = {}

    @torch.no_grad()
    def init_weights(self, std: float = 0.02):
        nn.init.normal_(self.router, std=std)
        self.experts.init_weights(std)
        if self.shared is not None:
            nn.init.normal_(self.shared.gate_up.weight, std=std)
            nn.init.normal_(self.shared.down.weight, std=std)
        if self.shared_gate is not None:
            nn.init.zeros_(self.shared_gate.weight)

    def _record(self, idx, scores, logits_for_z=None):
        load = torch.bincount(idx.flatten(), minlength=self.n_experts).float()
        self._cumulative_expert_load = load if self._cumulative_expert_load is None else self._cumulative_expert_load + load
        frac = load / load.sum().clamp_min(1)
        prob = scores.mean(0) / scores.mean(0).sum().clamp_min(1e-20)
        self.last_metrics = {"aux_loss": self.n_experts * (frac * prob).sum(), "load": load}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, self.dim)
        w, idx, scores = route(x2, self.router, self.e_score_correction_bias, top_k=self.top_k, score=self.score,
                               route_scale=self.route_scale)
        self._record(idx, scores)
        tok = torch.arange(x2.size(0), device=x.device).repeat_interleave(self.top_k)
        y = self.experts(x2[tok], idx.flatten(), w.flatten()[:, None])
        routed = torch.zeros(x2.shape, dtype=torch.float32, device=x.device).index_add_(0, tok, y)
        out = routed
        if self.shared is not None:
            s = self.shared(x2).float()
            if self.shared_gate is not None:
                s = s * torch.sigmoid(self.shared_gate(x2).float())
            out = out + s
        return out.to(x.dtype).reshape(shape)


# ------------------------------------------------------------------------------------------------
# expert parallelism
# ------------------------------------------------------------------------------------------------
class _Exchange(torch.autograd.Function):
    @staticmethod
    def forward(ctx, values, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = values.new_empty((sum(recv), *values.shape[1:]))
        dist.all_to_all_single(out, values.contiguous(), recv, send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send), *g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), ctx.send, ctx.recv, group=ctx.group)
        return out, None, None, None


def exchange(values, send, recv, group):
    return _Exchange.apply(values, send, recv, group)


def exchange_layout(destinations: torch.Tensor, group):
    size = dist.get_world_size(group)
    counts = torch.bincount(destinations, minlength=size)
    incoming = torch.empty_like(counts)
    dist.all_to_all_single(incoming, counts, group=group)
    return destinations.argsort(stable=True), counts.tolist(), incoming.tolist()


class ExpertParallelMoE(nn.Module):
    """Each rank owns ``E / ep`` experts; tokens travel to the owner and come back."""

    def __init__(self, dim: int, inter: int, n_experts: int, top_k: int, group, *, score="sqrt_softplus",
                 route_scale: float = 1.0, swiglu_limit: float | None = None, n_shared: int = 1):
        super().__init__()
        self.group = group
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if n_experts % self.size:
            raise ValueError("expert count must divide EP size")
        self.dim, self.n_experts, self.top_k, self.score, self.route_scale = dim, n_experts, top_k, score, route_scale
        self.local_experts = n_experts // self.size
        self.first = self.rank * self.local_experts
        self.router = nn.Parameter(torch.empty(n_experts, dim))
        self.register_buffer("e_score_correction_bias", torch.zeros(n_experts, dtype=torch.float32))
        self.experts = GroupedExperts(self.local_experts, dim, inter, swiglu_limit=swiglu_limit)
        self.shared = SwiGLU(dim, inter * n_shared, swiglu_limit) if n_shared else None
        self._cumulative_expert_load = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, self.dim)
        w, idx, _ = route(x2, self.router, self.e_score_correction_bias, top_k=self.top_k, score=self.score,
                          route_scale=self.route_scale)
        load = torch.bincount(idx.flatten(), minlength=self.n_experts).float()
        self._cumulative_expert_load = load if self._cumulative_expert_load is None else self._cumulative_expert_load + load
        ids = idx.flatten()
        order, send, recv = exchange_layout(ids // self.local_experts, self.group)
        tok = torch.arange(x2.size(0), device=x.device).repeat_interleave(self.top_k)[order]
        got_ids = exchange(ids[order], send, recv, self.group)
        got_x = exchange(x2[tok], send, recv, self.group)
        got_w = exchange(w.flatten()[order, None], send, recv, self.group)
        # an empty receiver still takes part in every reverse collective
        y = got_x.float() * 0 + got_w * 0
        if got_ids.numel():
            y = y + self.experts(got_x, got_ids, got_w, first_expert=self.first)
        back = exchange(y, recv, send, self.group)
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(order.numel(), device=order.device)
        expert_order = idx.argsort(dim=-1)
        slots = torch.arange(x2.size(0), device=x.device) * self.top_k
        routed = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
        for k in range(self.top_k):                       # ascending expert id: deterministic FP32 sum
            routed = routed + back[inverse[slots + expert_order[:, k]]]
        if self.shared is not None:
            routed = routed + self.shared(x2).float()
        return routed.to(x.dtype).reshape(shape)


# ------------------------------------------------------------------------------------------------
# aux-free load balancing
# ------------------------------------------------------------------------------------------------
def bias_correction(load: torch.Tensor, rate: float, *, proportional: bool = False) -> torch.Tensor:
    mean = load.float().mean()
    if proportional:
        change = ((mean - load.float()) / mean.clamp_min(1e-12)).clamp(-5.0, 1.0) * rate
        return change - change.mean()
    return (mean - load).sign() * rate


@torch.no_grad()
def balance_routers(gates, rate: float, *, proportional: bool = False, group=None) -> dict:
    if not gates or rate <= 0:
        raise ValueError("active learned routers and positive balance rate required")
    loads = []
    for g in gates:
        if g._cumulative_expert_load is None:
            raise ValueError("router load was not collected")
        loads.append(g._cumulative_expert_load.detach().float().clone())
    matrix = torch.stack(loads)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(matrix, group=group)
    cvs, dead, windows, sizes = [], [], [], []
    for g, load in zip(gates, matrix):
        bias = g.e_score_correction_bias
        if bias.dtype != torch.float32:
            raise ValueError("routing bias must retain FP32 precision")
        bias.add_(bias_correction(load, rate, proportional=proportional))
        g._cumulative_expert_load = None
        cvs.append(float(load.std() / load.mean().clamp_min(1)))
        dead.append(float((load == 0).float().mean()))
        if not hasattr(g, "_recent_expert_usage"):
            g._recent_expert_usage = deque(maxlen=20)
        g._recent_expert_usage.append((load > 0).clone())
        windows.append(float((~torch.stack(tuple(g._recent_expert_usage)).any(0)).float().mean()))
        sizes.append(len(g._recent_expert_usage))
    return {"router_load_cv_mean": sum(cvs) / len(cvs), "router_load_cv_max": max(cvs),
            "router_dead_fraction_mean": sum(dead) / len(dead), "router_dead_fraction_max": max(dead),
            "router_cv_per_layer": cvs, "router_unused_fraction_per_layer": dead,
            "router_unused_fraction_window": sum(windows) / len(windows),
            "router_worst_unused_fraction_window": max(windows), "router_usage_window_updates": min(sizes)}
