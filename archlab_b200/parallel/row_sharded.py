"""Row-sharded frozen lookup tables (the FP8 Engram memories of the V4.1 family).

A table of ``num_embeddings`` rows is stored as e4m3 values with one ue8m0 (power-of-two) scale per group of 32
columns and cut into ``ceil(num_embeddings / world)`` rows per rank.  A lookup sends every id to the rank that owns
its row, de-quantises the rows there and sends bf16 values back, in the order of the request
(src/archlab/automodel/deepseek_v41_parallel.py:113-142).  The table is frozen: no gradient flows.

The exchange is ``all_to_all_single`` (NCCL or gloo); the owner-side gather + de-quantisation is one kernel on a GPU
(``nga_gather_dequant_fp8``) and the PyTorch statement of it elsewhere.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import native

GROUP = 32
_vp, _i, _ll = C.c_void_p, C.c_int, C.c_longlong
native.register_signature("nga_gather_dequant_fp8", [_vp, _vp, _vp, _vp, _ll, _ll, _i, _vp])


def quantize_rows_e8m0(table: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[rows, dim] -> (e4m3 values as uint8 [rows, dim], biased exponents uint8 [rows, dim / 32])."""
    rows, dim = table.shape
    if dim % GROUP:
        raise ValueError("the table width must be a multiple of 32 (one scale per 32 columns)")
    g = table.float().view(rows, dim // GROUP, GROUP)
    amax = g.abs().amax(-1).clamp_min(1e-30)
    e = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    q = (g * torch.exp2(-e).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(rows, dim).view(torch.uint8), (e + 127).to(torch.uint8)


def dequantize_rows_e8m0(values: torch.Tensor, exponents: torch.Tensor) -> torch.Tensor:
    v = values.view(torch.float8_e4m3fn).float()
    s = torch.exp2(exponents.float() - 127.0).repeat_interleave(GROUP, -1)
    return (v * s).bfloat16()


class RowShardedTable(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, *, group=None, device=None):
        super().__init__()
        if embedding_dim % GROUP:
            raise ValueError("row-sharded tables carry one scale per 32 columns")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.rows = -(-num_embeddings // self.world)
        self.weight = nn.Parameter(torch.zeros(self.rows, embedding_dim, dtype=torch.uint8, device=device), requires_grad=False)
        self.scale = nn.Parameter(torch.full((self.rows, embedding_dim // GROUP), 127, dtype=torch.uint8, device=device),
                                  requires_grad=False)

    @torch.no_grad()
    def load_full(self, table: torch.Tensor) -> None:
        """Quantises this rank's row block of a full-precision table (tests, conversions)."""
        lo = self.rank * self.rows
        block = torch.zeros(self.rows, self.embedding_dim, dtype=torch.float32)
        part = table[lo:lo + self.rows].float().cpu()
        block[: part.size(0)] = part
        q, e = quantize_rows_e8m0(block)
        self.weight.copy_(q)
        self.scale.copy_(e)

    def _local_rows(self, local_ids: torch.Tensor) -> torch.Tensor:
        if local_ids.numel() == 0:
            return torch.empty(0, self.embedding_dim, dtype=torch.bfloat16, device=local_ids.device)
        if local_ids.is_cuda and native.available():
            out = torch.empty(local_ids.numel(), self.embedding_dim, dtype=torch.bfloat16, device=local_ids.device)
            rc = native.lib().nga_gather_dequant_fp8(self.weight.data_ptr(), self.scale.data_ptr(), local_ids.contiguous().data_ptr(),
                                                     out.data_ptr(), local_ids.numel(), self.rows, self.embedding_dim,
                                                     native.stream_ptr())
            native.check(rc, "nga_gather_dequant_fp8")
            return out
        return dequantize_rows_e8m0(self.weight[local_ids], self.scale[local_ids])

    @torch.no_grad()
    def forward(self, indices: torch.Tensor) -> torch.Tensor:
        ids = indices.reshape(-1).long()
        if ids.numel() and bool(((ids < 0) | (ids >= self.num_embeddings)).any()):
            raise ValueError("lookup outside the table")
        if self.world == 1:
            return self._local_rows(ids).view(*indices.shape, self.embedding_dim)
        owner = ids // self.rows
        order = owner.argsort(stable=True)
        send = torch.bincount(owner, minlength=self.world)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        send_l, recv_l = send.tolist(), recv.tolist()
        wanted = ids.new_empty(sum(recv_l))
        dist.all_to_all_single(wanted, ids[order].contiguous(), recv_l, send_l, group=self.group)
        rows = self._local_rows(wanted - self.rank * self.rows)
        back = rows.new_empty(sum(send_l), self.embedding_dim)
        dist.all_to_all_single(back, rows.contiguous(), send_l, recv_l, group=self.group)
        out = torch.empty_like(back)
        out[order] = back
        return out.view(*indices.shape, self.embedding_dim)
