"""Grouped linear layer: one tcgen05 GEMM launch for all experts of a rank.

Rows are sorted by expert and every expert's segment is padded to a multiple of 256 rows, so that each
256-row tile of the pair-CTA GEMM belongs to one expert; a small int table names the expert of every
tile and the kernel offsets its B coordinate into the stacked weights.  Forward and input gradient are
one launch each; weight gradients are per-expert ``dY_e^T X_e`` products on the same kernel (their
reduction lengths differ per expert).  Replaces a per-expert loop of 2 * E launches per layer; the
reference reaches TE ``GroupedLinear`` for this (src/archlab/architectures/qwen38_flash_next.py:184-202).
Off the GPU the per-expert loop runs.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import gemm as G
from . import native

TILE = 256
_vp, _i, _ll = C.c_void_p, C.c_int, C.c_longlong
native.register_signature("nga_gemm2_grouped_bf16", [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _i, _vp, _vp])
native.register_signature("nga_gemm2_grouped_wgrad_bf16", [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _vp, _vp])


def padded_sizes(counts: torch.Tensor) -> torch.Tensor:
    return (counts + TILE - 1) // TILE * TILE


def _launch(a, w_stack, tile_group, groups, n_out, k_red, b_mn):
    out = torch.empty(a.size(0), n_out, dtype=torch.bfloat16, device=a.device)
    rc = native.lib().nga_gemm2_grouped_bf16(a.data_ptr(), w_stack.data_ptr(), out.data_ptr(), tile_group.data_ptr(), groups, a.size(0),
                                             n_out, k_red, a.stride(0), w_stack.stride(0), out.stride(0), int(b_mn),
                                             native.status_word(a.device).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_gemm2_grouped_bf16")
    return out


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, tile_group, real, padded, fp8=False):
        E, N, K = w.shape
        ctx.save_for_backward(x, w, tile_group)
        ctx.seg = (real, padded)
        if fp8:
            # forward product in block-scaled FP8 (rows 1 x 128, expert weights 128 x 128 blocks); the backward below
            # is taken straight through the rounding against the bf16 operands
            from . import blockscaled as bs

            return bs.grouped_gemm(bs.quantize_fp8(x, 128), bs.quantize_fp8(w.view(E * N, K), -128), tile_group, E, N)
        return _launch(x, w.view(E * N, K), tile_group, E, N, K, False)

    @staticmethod
    def backward(ctx, dy):
        x, w, tile_group = ctx.saved_tensors
        real, padded = ctx.seg
        E, N, K = w.shape
        dy = dy.contiguous()
        dx = _launch(dy, w.view(E * N, K), tile_group, E, K, N, True)          # dY W_e: B read MN-major, reduction over N
        dw = torch.zeros_like(w)
        s0 = 0
        for e, (n, npad) in enumerate(zip(real, padded)):
            if n:
                dw[e] = G.gemm(dy[s0:s0 + n], x[s0:s0 + n], a_mn=True, b_mn=True)     # dY_e^T X_e
            s0 += npad
        return dx, dw, None, None, None, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, real: list[int], padded: list[int],
                   fp8: bool = False) -> torch.Tensor:
    """x [sum(padded), K] (rows sorted by expert, segments padded to 256), w [E, N, K] -> [sum(padded), N].
    Rows in the padding produce unspecified values.  ``fp8``: the forward product runs on the block-scaled FP8 GEMM
    (needs N and K to be multiples of 128); gradients are straight-through in bf16."""
    E, N, K = w.shape
    if x.size(0) == 0:
        # keeps the weights AND the (empty) input in the graph: the input's producer may be a collective autograd function
        # (expert dispatch) whose backward every rank must run, rows or no rows
        return x.new_zeros(0, N) + (0 * w.sum() + 0 * x.sum()).to(x.dtype)
    if x.is_cuda and x.dtype == torch.bfloat16 and native.available() and K % 8 == 0 and N % 64 == 0 and K % 64 == 0:
        return _GroupedLinear.apply(x.contiguous(), w.to(x.dtype).contiguous(), tile_group, real, padded,
                                    bool(fp8 and N % 128 == 0 and K % 128 == 0))
    outs, s0 = [], 0
    for e, npad in enumerate(padded):
        outs.append(x[s0:s0 + npad] @ w[e].to(x.dtype).t())
        s0 += npad
    return torch.cat(outs, 0) if outs else x.new_zeros(0, N)


def tile_groups(padded: list[int], device) -> torch.Tensor:
    reps = torch.tensor([p // TILE for p in padded], device=device)
    return torch.repeat_interleave(torch.arange(len(padded), device=device, dtype=torch.int32), reps).contiguous()


# ------------------------------------------------------------------------------------------------
# Device-planned form: nothing about the segment sizes is known on the host
# ------------------------------------------------------------------------------------------------
def device_plan(padded: torch.Tensor, bound_rows: int):
    """From the padded segment sizes (device int tensor, multiples of 256) and a fixed row bound: the group of every
    256-row tile of the bound (-1 past the used rows) and the [first, last) 64-row block of every group.  All on the
    device; ``bound_rows`` is a host constant (a multiple of 256) that the caller guarantees (and checks) to suffice."""
    if bound_rows % TILE:
        raise ValueError("the row bound must be a multiple of 256")
    ends = padded.cumsum(0)
    starts = ends - padded
    tile_first = torch.arange(bound_rows // TILE, device=padded.device, dtype=ends.dtype) * TILE
    group = torch.searchsorted(ends, tile_first, right=True)
    tile_group = torch.where(tile_first < ends[-1], group, torch.full_like(group, -1)).to(torch.int32).contiguous()
    kb_range = torch.stack([starts // 64, ends // 64], 1).to(torch.int32).contiguous()
    return tile_group, kb_range


class _GroupedLinearDevice(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, tile_group, kb_range, fp8=False, out=None):
        E, N, K = w.shape
        ctx.save_for_backward(x, w, tile_group, kb_range)
        if fp8:
            from . import blockscaled as bs

            y = bs.grouped_gemm(bs.quantize_fp8(x, 128), bs.quantize_fp8(w.view(E * N, K), -128), tile_group, E, N)
            return y if out is None else out.copy_(y)
        y = torch.empty(x.size(0), N, dtype=torch.bfloat16, device=x.device) if out is None else out
        rc = native.lib().nga_gemm2_grouped_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), tile_group.data_ptr(), E, x.size(0), N, K,
                                                 x.stride(0), K, y.stride(0), 0, native.status_word(x.device).data_ptr(), native.stream_ptr())
        native.check(rc, "nga_gemm2_grouped_bf16")
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, tile_group, kb_range = ctx.saved_tensors
        E, N, K = w.shape
        dy = dy.contiguous()
        dx = torch.zeros(x.size(0), K, dtype=torch.bfloat16, device=x.device)       # skipped tiles stay zero
        rc = native.lib().nga_gemm2_grouped_bf16(dy.data_ptr(), w.data_ptr(), dx.data_ptr(), tile_group.data_ptr(), E, dy.size(0), K, N,
                                                 dy.stride(0), K, dx.stride(0), 1, native.status_word(x.device).data_ptr(), native.stream_ptr())
        native.check(rc, "nga_gemm2_grouped_bf16")
        dw = torch.zeros_like(w)                                                     # groups without rows are skipped
        rc = native.lib().nga_gemm2_grouped_wgrad_bf16(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), kb_range.data_ptr(), E, dy.size(0), N, K,
                                                       dy.stride(0), x.stride(0), native.status_word(x.device).data_ptr(), native.stream_ptr())
        native.check(rc, "nga_gemm2_grouped_wgrad_bf16")
        return dx, dw, None, None, None, None


def grouped_linear_device(x: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, kb_range: torch.Tensor, *, fp8: bool = False,
                          out: torch.Tensor | None = None) -> torch.Tensor:
    """``grouped_linear`` with the segment layout on the device (``device_plan``): ``x`` has the fixed bound of rows, tiles
    past the used rows are skipped by the kernels (their output rows are unspecified in the forward and zero in the
    data gradient) and the weight gradient is one launch whose reduction ranges come from ``kb_range``.  Rows of the
    padding inside a segment must be finite in ``x`` and zero in the incoming gradient.  bf16 CUDA only; N and K
    multiples of 256 resp. 64."""
    E, N, K = w.shape
    if not (x.is_cuda and x.dtype == torch.bfloat16 and native.available() and K % 64 == 0 and N % 64 == 0 and x.size(0) % TILE == 0):
        raise ValueError("grouped_linear_device needs bf16 CUDA operands, K and N multiples of 64 and a 256-row bound")
    return _GroupedLinearDevice.apply(x.contiguous(), w.to(x.dtype).contiguous(), tile_group, kb_range,
                                      bool(fp8 and N % 128 == 0 and K % 128 == 0), out)
