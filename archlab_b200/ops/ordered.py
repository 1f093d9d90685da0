"""Order-fixed fp32 sums for paths that promise bit-reproducible results.

Floating-point addition is not associative, so a sum whose order depends on thread scheduling (atomics, ``index_add_``
on a GPU with repeated destinations) changes bits from run to run.  Two reductions with a FIXED order:

* ``ordered_index_sum(destination, indices, values)``: rows of ``values`` that share an index are added in their input
  order (stable sort, one segment reduction per destination, a single write per destination row).
* ``ordered_permutation_sum(values, positions)``: the expert-combine pattern.  ``positions[t, k]`` is the row of
  ``values`` that holds token ``t``'s k-th expert output (-1: none); every row of ``values`` is used exactly once.  The
  result is ``sum_k values[positions[t, k]]`` accumulated slot by slot in fp32 -- slot order is the order the caller
  chose (ascending expert id).  Work proceeds in row chunks so the fp32 temporary stays bounded; the backward is a pure
  permutation (each dispatched row receives exactly one gradient row), written with ``index_copy_`` into an
  uninitialised buffer instead of adding zero-filled gradients per slot.
(Reference: src/archlab/architectures/ordered_reduction.py:6-13, ordered_scatter.py:12-60.)
"""
from __future__ import annotations

import torch


def ordered_index_sum(destination: torch.Tensor, indices: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    if indices.numel() == 0:
        return destination
    order = torch.sort(indices, stable=True).indices
    keys, lengths = torch.unique_consecutive(indices[order], return_counts=True)
    sums = torch.segment_reduce(values[order].to(destination.dtype), "sum", lengths=lengths)
    destination[keys] += sums                                   # keys are unique: one write per row, no accumulation race
    return destination


class _PermutationSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, values, positions, chunk_rows):
        tokens, slots = positions.shape
        out = torch.zeros(tokens, values.shape[1], dtype=torch.float32, device=values.device)
        for start in range(0, tokens, chunk_rows):
            block = positions[start:start + chunk_rows]
            acc = out[start:start + chunk_rows]
            for k in range(slots):                               # fixed slot order = fixed summation order
                rows = block[:, k]
                present = rows >= 0
                acc += values[rows.clamp_min(0)].float() * present[:, None]
        ctx.save_for_backward(positions)
        ctx.meta = (values.shape, values.dtype, chunk_rows)
        return out

    @staticmethod
    def backward(ctx, grad):
        (positions,) = ctx.saved_tensors
        shape, dtype, chunk_rows = ctx.meta
        if not ctx.needs_input_grad[0]:
            return None, None, None
        out = torch.empty(shape, dtype=dtype, device=grad.device)
        token, slot = torch.nonzero(positions >= 0, as_tuple=True)
        for part_t, part_s in zip(token.split(chunk_rows), slot.split(chunk_rows)):
            out.index_copy_(0, positions[part_t, part_s], grad[part_t].to(dtype))
        return out, None, None


def ordered_permutation_sum(values: torch.Tensor, positions: torch.Tensor, *, chunk_rows: int = 8192, validate: bool = True) -> torch.Tensor:
    if (values.ndim != 2 or positions.ndim != 2 or positions.dtype not in (torch.int32, torch.int64) or values.device != positions.device
            or not values.is_floating_point() or type(chunk_rows) is not int or chunk_rows < 1):
        raise ValueError("expected floating rows, integral positions and a positive chunk size")
    positions = positions.long()
    if validate:
        used = positions[positions >= 0].sort().values
        if bool((positions < -1).any()) or used.numel() != values.shape[0] or not torch.equal(used, torch.arange(values.shape[0], device=values.device)):
            raise ValueError("positions must be a permutation of every source row, with -1 padding")
    return _PermutationSum.apply(values, positions, chunk_rows)
