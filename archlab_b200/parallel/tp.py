"""Tensor parallelism with sequence parallelism: linear layers whose collective is fused into the
GEMM kernel over NVLink peer memory.

* ``ag_gemm``   : Y = all_gather_rows(X_shard) @ W^T   (column-parallel forward; row-parallel dgrad).
  A few clusters of the GEMM kernel pull the remote row shards once into a local gathered buffer
  (bulk copies; about a dozen clusters keep an NVLink port busy) and flag 128-row blocks as they
  land, while the tensor cores start on this rank's own rows.
* ``gemm_rs``   : reduce_scatter_rows(A @ W^T)          (row-parallel forward; column-parallel dgrad).
  Every output tile is stored straight into the staging slot of the rank that owns those rows
  (remote owners first); the owner then sums the ``world`` slots (optionally with the residual).

They replace Megatron's ``TEColumnParallelLinear`` / ``TERowParallelLinear`` under sequence
parallelism (src/archlab/megatron/qwen38_flash_next_model.py:179-205), whose collectives are
separate NCCL all-gather / reduce-scatter calls.  On CPU (gloo) or without the native library the
same functions run the decomposed gather + matmul / matmul + reduce-scatter, which is also the
test oracle.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import native
from . import collectives as coll

_vp, _i, _ll = C.c_void_p, C.c_int, C.c_longlong
native.register_signature("nga_tp_gemm_bf16", [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _i, _i, _i, _i, _vp, _vp, _vp,
                                               _i, _i, _vp, _vp, _vp])
native.register_signature("nga_tp_reduce_slots", [_vp, _vp, _vp, _i, _ll, _i, _ll, _ll, _ll, _vp])
native.register_signature("nga_tp_gemm_push_bf16", [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp])
native.register_signature("nga_tp_gemm_rs_reduce_bf16", [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i, _vp, _vp,
                                                         _i, _vp, _vp])


class TPGroup:
    """Symmetric buffers and barriers of one tensor-parallel group for a fixed problem geometry:
    ``rows`` sequence rows per rank, activations up to ``max_k`` wide, outputs up to ``max_n`` wide."""

    def __init__(self, rows: int, max_k: int, max_n: int, device, group=None, copy_clusters: int = 12, push: bool | None = None):
        """``push``: owner-push all-gather and in-kernel reduce-scatter (one launch per op, no barrier kernels); False
        selects the pull form (copy clusters, barrier + separate slot reduction), kept for comparison."""
        from .symm import PeerBarrier, symm_empty, symm_zeros

        self.group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if rows % 256:
            raise ValueError("rows per rank must be a multiple of 256")
        self.rows, self.max_k, self.max_n, self.device = rows, max_k, max_n, device
        self.copy_clusters = copy_clusters
        # all-gather source, double-buffered: a peer may still be pulling call k's shard while this rank
        # already writes the shard of call k + 1 (the barrier of call k + 1 orders everything older)
        self.x_shard = symm_empty((2 * rows * max_k,), torch.bfloat16, device, self.group)
        self.stage = symm_empty((self.world * rows * max_n,), torch.bfloat16, device, self.group)  # RS slots
        self.gathered = torch.empty(self.world * rows * max_k, dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros(self.world * rows // 128, dtype=torch.int32, device=device)
        self.epoch = 0
        self.barrier = PeerBarrier(device, self.group)
        # owner-push / in-epilogue reduction measured faster than the copy-cluster forms at two ranks (0.13 / 0.147 against
        # 0.154 / 0.157 ms) and slower at four (0.272 / 0.274 against 0.261 / 0.244 ms: three peers' pushes occupy every CTA)
        self.push = push = (self.world == 2) if push is None else push
        if push:
            # both directions alternate between two buffers from call to call: a rank can be at most one call ahead of a
            # peer (finishing a call needs every peer's data of that call), so the buffer of call k is free at call k + 2
            self.gathered2 = symm_empty((2 * self.world * rows * max_k,), torch.bfloat16, device, self.group)
            self.block_flags = symm_zeros((self.world * rows // 128,), torch.int32, device, self.group)
            self.stage2 = symm_empty((2 * self.world * rows * max_n,), torch.bfloat16, device, self.group)
            self.counters = symm_zeros((rows // 256 * ((max_n + 255) // 256 + 1),), torch.int32, device, self.group)
            self.push_epoch = 0
            self.rs_calls = 0
            self._rs_shape = None
            torch.cuda.synchronize(device)
            self.barrier()                       # every rank's flags and counters are zero before anyone writes to them
            torch.cuda.synchronize(device)

    def shard_view(self, k: int, epoch: int | None = None) -> torch.Tensor:
        """The shard buffer the call with this epoch (default: the next call) reads; a producer can write
        its output straight into it and pass it to ``ag_gemm`` to skip the staging copy."""
        half = ((self.epoch + 1) if epoch is None else epoch) & 1
        base = half * self.rows * self.max_k
        return self.x_shard.tensor[base: base + self.rows * k].view(self.rows, k)

    def gathered_view(self, k: int) -> torch.Tensor:
        if self.push:                            # the buffer the latest call filled
            base = (self.push_epoch & 1) * self.world * self.rows * self.max_k
            return self.gathered2.tensor[base: base + self.world * self.rows * k].view(self.world * self.rows, k)
        return self.gathered[: self.world * self.rows * k].view(self.world * self.rows, k)


def ag_gemm(tp: TPGroup, x_shard: torch.Tensor, w: torch.Tensor, *, w_mn: bool = False,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """x_shard [rows, K] (this rank's sequence slice) -> [world*rows, N] = gather(x) @ (w^T or w).
    ``w`` is [N, K] (``w_mn=False``) or [K, N] (``w_mn=True``).  The gathered activations stay in
    ``tp.gathered_view(K)`` for the weight-gradient GEMM."""
    rows, K = x_shard.shape
    N = w.size(1) if w_mn else w.size(0)
    M = tp.world * rows
    if rows != tp.rows or K > tp.max_k:
        raise ValueError("geometry does not match the TP group")
    if tp.push:
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x_shard.device)
        x_shard = x_shard.contiguous()
        tp.push_epoch += 1
        base = (tp.push_epoch & 1) * tp.world * tp.rows * tp.max_k
        rc = native.lib().nga_tp_gemm_push_bf16(
            x_shard.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, w.stride(0), out.stride(0), int(w_mn), tp.rank, tp.world,
            rows, tp.gathered2.ptr_array(base), tp.block_flags.ptr_array(), tp.push_epoch,
            native.status_word(x_shard.device).data_ptr(), native.stream_ptr())
        native.check(rc, "nga_tp_gemm_push_bf16")
        return out
    src = tp.shard_view(K)
    if x_shard.data_ptr() != src.data_ptr():
        src.copy_(x_shard)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x_shard.device)
    tp.barrier()                                   # every rank's shard for this epoch is written
    tp.epoch += 1
    rc = native.lib().nga_tp_gemm_bf16(
        None, w.data_ptr(), out.data_ptr(), M, N, K, w.stride(0), out.stride(0), int(w_mn), 1, tp.rank, tp.world, rows,
        tp.x_shard.ptr_array((tp.epoch & 1) * tp.rows * tp.max_k), tp.gathered.data_ptr(), tp.flags.data_ptr(),
        tp.epoch, tp.copy_clusters, None, native.status_word(x_shard.device).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_tp_gemm_bf16(all-gather)")
    return out


def gemm_rs(tp: TPGroup, a: torch.Tensor, w: torch.Tensor, *, w_mn: bool = False, resid: torch.Tensor | None = None,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """a [world*rows, K_local] -> this rank's [rows, N] slice of sum_over_ranks(a @ w^T) (+ resid)."""
    M, K = a.shape
    N = w.size(1) if w_mn else w.size(0)
    if M != tp.world * tp.rows or N > tp.max_n:
        raise ValueError("geometry does not match the TP group")
    if out is None:
        out = torch.empty(tp.rows, N, dtype=torch.bfloat16, device=a.device)
    if tp.push and N % 32 == 0 and (resid is None or resid.stride(0) % 8 == 0):
        if tp._rs_shape not in (None, N):
            raise ValueError("one TP group reduces outputs of one width (the arrival counters are indexed by tile)")
        tp._rs_shape = N
        tp.rs_calls += 1
        base = (tp.rs_calls & 1) * tp.world * tp.rows * tp.max_n
        rc = native.lib().nga_tp_gemm_rs_reduce_bf16(
            a.data_ptr(), w.data_ptr(), out.data_ptr(), None if resid is None else resid.data_ptr(), M, N, K, w.stride(0),
            out.stride(0), 0 if resid is None else resid.stride(0), int(w_mn), tp.rank, tp.world, tp.rows,
            tp.stage2.ptr_array(base), tp.counters.ptr_array(), tp.rs_calls, native.status_word(a.device).data_ptr(),
            native.stream_ptr())
        native.check(rc, "nga_tp_gemm_rs_reduce_bf16")
        return out
    tp.barrier()                                   # every owner has consumed its slots from the previous call
    rc = native.lib().nga_tp_gemm_bf16(
        a.data_ptr(), w.data_ptr(), None, M, N, K, w.stride(0), N, int(w_mn), 2, tp.rank, tp.world, tp.rows,
        None, None, None, 0, 0, tp.stage.ptr_array(), native.status_word(a.device).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_tp_gemm_bf16(reduce-scatter)")
    tp.barrier()                                   # all partial tiles have landed
    rc = native.lib().nga_tp_reduce_slots(tp.stage.tensor.data_ptr(), None if resid is None else resid.data_ptr(),
                                          out.data_ptr(), tp.world, tp.rows, N, N, 0 if resid is None else resid.stride(0),
                                          out.stride(0), native.stream_ptr())
    native.check(rc, "nga_tp_reduce_slots")
    return out


# ------------------------------------------------------------------------------------------------
# decomposed forms (CPU / gloo path and the oracles of the fused kernels)
# ------------------------------------------------------------------------------------------------
def ag_gemm_reference(x_shard: torch.Tensor, w: torch.Tensor, group=None, *, w_mn: bool = False) -> torch.Tensor:
    world = coll.world_size(group)
    parts = [torch.empty_like(x_shard) for _ in range(world)]
    if world > 1:
        dist.all_gather(parts, x_shard.contiguous(), group=group)
    else:
        parts = [x_shard]
    x = torch.cat(parts, 0).float()
    return (x @ (w.float() if w_mn else w.float().t())).to(x_shard.dtype)


def gemm_rs_reference(a: torch.Tensor, w: torch.Tensor, group=None, *, w_mn: bool = False,
                      resid: torch.Tensor | None = None) -> torch.Tensor:
    world, rank = coll.world_size(group), coll.rank(group)
    y = a.float() @ (w.float() if w_mn else w.float().t())
    if world > 1:
        dist.all_reduce(y, group=group)
    rows = y.size(0) // world
    out = y[rank * rows:(rank + 1) * rows]
    if resid is not None:
        out = out + resid.float()
    return out.to(a.dtype)
