"""Expert parallelism whose all-to-all is fused with the token permutation in kernels that read and
write peer memory directly (``csrc/moe.cu``).

Forward of one MoE layer on every rank:
  route -> counts exchanged (tiny all-gather) -> prefix sums give every (token, slot) its row in the
  owner's receive buffer -> ``push_rows`` writes the token rows straight into the owners' buffers
  (dispatch = all-to-all + permute, one kernel) -> device barrier -> per-expert tcgen05 GEMMs + clamped
  SwiGLU on contiguous expert segments -> device barrier -> ``pull_combine`` reads every token's k
  expert rows back from the owners and sums them, weighted, in ascending expert id (combine =
  all-to-all + un-permute + ordered fp32 sum, one kernel).
Backward uses the same two kernels as each other's adjoint.  The NCCL all-to-all form
(``models.moe.ExpertParallelMoE``; src/archlab/automodel/deepseek_v41_parallel.py:16-111) is the
baseline and the oracle.
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..models.moe import GroupedExperts, SwiGLU, route
from ..ops import block_ops, grouped
from ..ops import native
from ..ops.linear import linear

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
native.register_signature("nga_moe_push_rows", [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp])
native.register_signature("nga_moe_pull_combine", [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp])
native.register_signature("nga_swiglu_clamped", [_vp, _vp, _vp, _ll, _i, _f, _vp])


class EPBuffers:
    """Symmetric buffers of one expert-parallel group: token rows in, expert rows out, and the two
    gradient buffers of the backward pass; ``capacity`` rows of ``dim`` bf16 each."""

    def __init__(self, capacity: int, dim: int, device, group=None):
        from .symm import PeerBarrier, symm_empty

        self.group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        # `capacity` counts routed rows; every local expert's segment is padded to a 256-row tile on top of that
        capacity = capacity + 256 * 64
        self.capacity, self.dim = capacity, dim
        mk = lambda: symm_empty((capacity * dim,), torch.bfloat16, device, self.group)
        self.recv_x, self.y, self.g_y, self.g_x = mk(), mk(), mk(), mk()
        for sym in (self.recv_x, self.y, self.g_y, self.g_x):
            sym.tensor.zero_()             # rows of segment padding are read by the grouped GEMMs: they must be finite
        self.barrier = PeerBarrier(device, self.group)
        # [rows past the bound that a layer's grouped GEMMs run over, most padded rows any layer received]: device
        # counters, read once per step by the trainer
        self.counters = torch.zeros(2, dtype=torch.int64, device=device)
        self.adaptive_bound: int | None = None      # "auto" capacity: None = worst case until the first step was seen

    @property
    def overflow(self):
        return self.counters[0]

    def note_rows(self, padded_rows: torch.Tensor, bound: int) -> None:
        """Device-side bookkeeping of one layer call (no synchronisation)."""
        self.counters[0] += (padded_rows - bound).clamp_min(0)
        self.counters[1] = torch.maximum(self.counters[1], padded_rows)

    def check_overflow(self, margin: float = 1.5) -> dict:
        """Once per step (a small collective and one device -> host read): how many rows arrived past a bound since the
        last call (their tokens' expert contributions were dropped, as in capacity-factor routing) and the largest row
        count any layer of any rank saw; the adaptive bound moves to ``margin`` x that, identically on every rank."""
        if self.world > 1:
            both = self.counters.clone()
            dist.all_reduce(both[:1], group=self.group)
            dist.all_reduce(both[1:], op=dist.ReduceOp.MAX, group=self.group)
        else:
            both = self.counters
        over, peak = both.tolist()
        self.counters.zero_()
        if peak:
            self.adaptive_bound = min(self.capacity // 256 * 256, (int(margin * peak) + 255) // 256 * 256)
        return {"dropped_rows": int(over), "peak_rows": int(peak), "bound": self.adaptive_bound}

    def view(self, sym, n):
        return sym.tensor[: n * self.dim].view(n, self.dim)


def _p(t):
    return None if t is None else t.data_ptr()


def push_rows(rows, dst_rank, dst_row, sym, buf: EPBuffers, scale=None, src_row=None):
    n = dst_rank.numel()
    rc = native.lib().nga_moe_push_rows(_p(rows), _p(src_row), _p(dst_rank), _p(dst_row), _p(scale), sym.ptr_array(), buf.world,
                                        n, buf.dim, native.stream_ptr())
    native.check(rc, "nga_moe_push_rows")


def pull_combine(sym, buf: EPBuffers, rank, row, weight, T, k, gout=None, want_dweight=False, fp32_out=False):
    out = None if fp32_out else torch.empty(T, buf.dim, dtype=torch.bfloat16, device=rank.device)
    out32 = torch.empty(T, buf.dim, dtype=torch.float32, device=rank.device) if fp32_out else None
    dw = torch.empty(T, k, dtype=torch.float32, device=rank.device) if want_dweight else None
    rc = native.lib().nga_moe_pull_combine(sym.ptr_array(), buf.world, _p(rank), _p(row), _p(weight), _p(gout), _p(out), _p(out32),
                                           _p(dw), T, k, buf.dim, native.stream_ptr())
    native.check(rc, "nga_moe_pull_combine")
    return (out32 if fp32_out else out), dw


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, src_row, dst_rank, dst_row, n_recv, k, buf, keep=None):
        ctx.meta = (dst_rank, dst_row, x.size(0), k, buf, n_recv, keep)
        buf.barrier()                                           # receive buffers are free everywhere
        push_rows(x, dst_rank, dst_row, buf.recv_x, buf, src_row=src_row)
        buf.barrier()                                           # every row has landed
        return buf.view(buf.recv_x, n_recv).clone()

    @staticmethod
    def backward(ctx, g_recv):
        dst_rank, dst_row, T, k, buf, n_recv, keep = ctx.meta
        buf.barrier()
        buf.view(buf.g_x, n_recv).copy_(g_recv)
        buf.barrier()
        # slots of a token are adjacent; slots dropped at the owner's row bound carry no gradient
        dx, _ = pull_combine(buf.g_x, buf, dst_rank, dst_row, None if keep is None else keep.view(T, k), T, k)
        return dx, None, None, None, None, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_local, weight, rank_sorted, row_sorted, T, k, buf, masked=False):
        ctx.masked = masked
        n = y_local.size(0)
        buf.barrier()
        buf.view(buf.y, n).copy_(y_local)
        buf.barrier()
        out, _ = pull_combine(buf.y, buf, rank_sorted, row_sorted, weight, T, k)
        ctx.save_for_backward(y_local, weight, rank_sorted, row_sorted)
        ctx.meta = (T, k, buf)
        return out

    @staticmethod
    def backward(ctx, gout):
        y_local, weight, rank_sorted, row_sorted = ctx.saved_tensors
        T, k, buf = ctx.meta
        n = y_local.size(0)
        gout = gout.contiguous()
        buf.view(buf.g_y, n).zero_()        # rows of segment padding must be zero for the grouped weight gradient
        buf.barrier()
        buf.view(buf.y, n).copy_(y_local)                        # expert rows again, for d(weight)
        buf.barrier()
        _, dw = pull_combine(buf.y, buf, rank_sorted, row_sorted, None, T, k, gout=gout, want_dweight=True, fp32_out=True)
        if ctx.masked:
            dw = dw * (weight != 0)                               # dropped slots read rows the owner never computed
        src_row = torch.arange(T, device=gout.device, dtype=torch.int32).repeat_interleave(k)
        push_rows(gout, rank_sorted.flatten(), row_sorted.flatten(), buf.g_y, buf, scale=weight.flatten().contiguous(),
                  src_row=src_row)
        buf.barrier()
        gy = buf.view(buf.g_y, n).clone()
        return gy, dw, None, None, None, None, None, None


class FusedExpertParallelMoE(nn.Module):
    """Same parameters and semantics as ``models.moe.ExpertParallelMoE``; bf16 CUDA only."""

    def __init__(self, dim, inter, n_experts, top_k, buffers: EPBuffers, *, score="sqrt_softplus", route_scale=1.0,
                 swiglu_limit=None, n_shared=1, fp8: bool = False, capacity_factor: float | str | None = None):
        super().__init__()
        self.buf = buffers
        # capacity_factor f: the grouped GEMMs run over a fixed bound of f x (tokens x top_k) + padding rows whose layout
        # lives on the device, so the layer never synchronises with the host; "auto": the bound follows the largest row
        # count of the previous step (x 1.5; the worst case before the first step was seen); None: exact sizes read
        # back per call
        self.capacity_factor = None if os.environ.get("NGA_EP_HOST_PLAN") == "1" else capacity_factor
        self.fp8 = fp8                      # forward products of the expert and shared projections in block-scaled FP8
        self.size, self.rank = buffers.world, buffers.rank
        if n_experts % self.size:
            raise ValueError("expert count must divide EP size")
        self.dim, self.n_experts, self.top_k, self.score, self.route_scale = dim, n_experts, top_k, score, route_scale
        self.local_experts = n_experts // self.size
        self.first = self.rank * self.local_experts
        self.limit = swiglu_limit
        self.router = nn.Parameter(torch.empty(n_experts, dim))
        self.register_buffer("e_score_correction_bias", torch.zeros(n_experts, dtype=torch.float32))
        self.experts = GroupedExperts(self.local_experts, dim, inter, swiglu_limit=swiglu_limit)
        self.shared = SwiGLU(dim, inter * n_shared, swiglu_limit, fp8=fp8) if n_shared else None
        self._cumulative_expert_load = None

    def plan(self, idx: torch.Tensor):
        """Routing indices [T, k] -> where every slot lives in its owner's buffer, and this rank's segments."""
        T, k = idx.shape
        E, El, W = self.n_experts, self.local_experts, self.size
        flat = idx.flatten()
        counts = torch.zeros(E, dtype=torch.int64, device=idx.device).scatter_add_(0, flat, torch.ones_like(flat))   # bincount would sync
        allc = torch.empty(W, E, dtype=counts.dtype, device=idx.device)
        dist.all_gather_into_tensor(allc, counts, group=self.buf.group)
        per_e = allc.sum(0)                                                     # rows of expert e on its owner
        pad_e = grouped.padded_sizes(per_e)                                     # segments start on 256-row tiles
        seg_start = pad_e.view(W, El).cumsum(1) - pad_e.view(W, El)            # start of e's segment on its owner
        before_me = allc[: self.rank].sum(0)                                    # rows of e from lower source ranks
        base = seg_start.flatten() + before_me
        sorted_e, order = flat.sort(stable=True)
        group_start = (counts.cumsum(0) - counts)[sorted_e]
        within = torch.arange(flat.numel(), device=idx.device) - group_start
        dst_row = torch.empty_like(flat)
        dst_row[order] = base[sorted_e] + within
        dst_rank = flat // El
        mine = torch.stack([per_e[self.first:self.first + El], pad_e[self.first:self.first + El]])
        return dst_rank.int(), dst_row.int(), mine, counts

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, self.dim).contiguous()
        T, k = x2.size(0), self.top_k
        w, idx, _ = route(x2, self.router, self.e_score_correction_bias, top_k=k, score=self.score, route_scale=self.route_scale)
        dst_rank, dst_row, mine, counts = self.plan(idx)
        load = counts.float()
        self._cumulative_expert_load = load if self._cumulative_expert_load is None else self._cumulative_expert_load + load
        if self.capacity_factor is not None and self.experts.inter % 128 == 0 and self.dim % 256 == 0:
            return self._forward_device_planned(x2, w, idx, dst_rank, dst_row, mine, shape)
        seg, seg_pad = mine.tolist()                                              # host needs the GEMM extents
        n_recv = sum(seg_pad)
        if n_recv > self.buf.capacity:
            raise RuntimeError(f"expert receive buffer too small: {n_recv} rows > capacity {self.buf.capacity}")
        src_row = torch.arange(T, device=x.device, dtype=torch.int32).repeat_interleave(k)
        recv = _Dispatch.apply(x2, src_row, dst_rank, dst_row, n_recv, k, self.buf, None)
        # all local experts in ONE grouped GEMM per projection (rows in the 256-row padding are never read back)
        tiles = grouped.tile_groups(seg_pad, x.device)
        h = grouped.grouped_linear(recv, self.experts.gate_up, tiles, seg, seg_pad, fp8=self.fp8)
        y_local = grouped.grouped_linear(block_ops.swiglu(h, self.limit), self.experts.down, tiles, seg, seg_pad, fp8=self.fp8)
        # ascending expert id per token: deterministic summation order
        eo = idx.argsort(dim=-1)
        slots = (torch.arange(T, device=x.device) * k).unsqueeze(1) + eo
        rank_s, row_s, w_s = dst_rank[slots].contiguous(), dst_row[slots].contiguous(), w.gather(1, eo).float().contiguous()
        out = _Combine.apply(y_local, w_s, rank_s, row_s, T, k, self.buf, False)
        if self.shared is not None:
            out = out + self.shared(x2).to(out.dtype)
        return out.reshape(shape)

    def _forward_device_planned(self, x2, w, idx, dst_rank, dst_row, mine, shape):
        """No host synchronisation: a fixed row bound, tile -> expert and reduction-range tables on the device."""
        T, k = x2.size(0), self.top_k
        limit = self.buf.capacity // grouped.TILE * grouped.TILE
        if self.capacity_factor == "auto":
            bound = self.buf.adaptive_bound or limit
        else:
            bound = int(self.capacity_factor * T * k) + grouped.TILE * self.local_experts
        bound = min((bound + grouped.TILE - 1) // grouped.TILE * grouped.TILE, limit)
        tiles, kb_range = grouped.device_plan(mine[1], bound)
        self.buf.note_rows(mine[1].sum(), bound)
        # every rank uses the same bound (same token count, or the all-reduced adaptive bound), so the sender knows which
        # of its slots land past it: those are dropped (weight 0, no gradient), as in capacity-factor routing
        keep = (dst_row < bound).float()
        src_row = torch.arange(T, device=x2.device, dtype=torch.int32).repeat_interleave(k)
        recv = _Dispatch.apply(x2, src_row, dst_rank, dst_row, bound, k, self.buf, keep)
        h = grouped.grouped_linear_device(recv, self.experts.gate_up, tiles, kb_range, fp8=self.fp8)
        y_local = grouped.grouped_linear_device(block_ops.swiglu(h, self.limit), self.experts.down, tiles, kb_range, fp8=self.fp8)
        eo = idx.argsort(dim=-1)
        slots = (torch.arange(T, device=x2.device) * k).unsqueeze(1) + eo
        rank_s, row_s = dst_rank[slots].contiguous(), dst_row[slots].contiguous()
        w_s = (w.gather(1, eo).float() * keep[slots]).contiguous()
        self._last_keep = keep.view(T, k)
        out = _Combine.apply(y_local, w_s, rank_s, row_s, T, k, self.buf, True)
        if self.shared is not None:
            out = out + self.shared(x2).to(out.dtype)
        return out.reshape(shape)
