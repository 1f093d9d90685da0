"""Single-token (decode) 2-simplicial attention against paged key/value caches.

Every sequence owns a list of 128-position pages in four shared caches (short keys / values, long keys /
values; ``[num_pages * 128, Hkv * D]`` bf16).  ``simplicial_decode`` attends the newest token of each
sequence to its short window (w1) x long window (w2) of cached positions.  On CUDA the work runs in the
decode mode of the tcgen05 forward kernel: the 128 accumulator rows are the (query head of one KV group,
short key) pairs, the long-window tiles are exactly the pages named by the block table, fetched by TMA.
The PyTorch statement below is the oracle and the CPU path.  Takes the place of the reference's decode /
paged kernels used by its serving bridge (src/archlab/architectures/tilelang_attention.py:383-420,
simplicial_kernels.py paged forms).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import native

PAGE = 128
_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
native.register_signature("nga_simplicial_decode", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _i, _i, _i, _i, _i, _i,
                                                    _i, _i, _f, _vp, _vp])


class PagedSimplicialCache:
    def __init__(self, num_pages: int, n_kv_heads: int, head_dim: int, device, dtype=torch.bfloat16):
        self.num_pages, self.hkv, self.d = num_pages, n_kv_heads, head_dim
        mk = lambda: torch.zeros(num_pages * PAGE, n_kv_heads * head_dim, device=device, dtype=dtype)
        self.k1, self.k2, self.v1, self.v2 = mk(), mk(), mk(), mk()
        self.free = list(range(num_pages - 1, -1, -1))

    def allocate(self, n_positions: int) -> list[int]:
        need = (n_positions + PAGE - 1) // PAGE
        if need > len(self.free):
            raise RuntimeError("out of cache pages")
        return [self.free.pop() for _ in range(need)]

    def release(self, pages) -> None:
        self.free.extend(pages)

    def rows(self, pages: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Physical row of each logical position given one sequence's page list."""
        return pages[positions // PAGE].long() * PAGE + positions % PAGE

    @torch.no_grad()
    def write(self, pages: torch.Tensor, start: int, k1, k2, v1, v2) -> None:
        """k*/v* [n, Hkv, D]: positions start .. start + n - 1 of one sequence."""
        n = k1.size(0)
        r = self.rows(pages, torch.arange(start, start + n, device=pages.device))
        for dst, src in ((self.k1, k1), (self.k2, k2), (self.v1, v1), (self.v2, v2)):
            dst[r] = src.reshape(n, -1).to(dst.dtype)


def simplicial_decode_reference(q, cache: PagedSimplicialCache, block_table, seq_lens, w1: int, w2: int, scale=None):
    """q [B, Hq, D] -> [B, Hq, D] in fp32: joint softmax over the valid (short, long) pairs of the last position."""
    B, Hq, D = q.shape
    g = Hq // cache.hkv
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out = torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device)
    for b in range(B):
        L = int(seq_lens[b])
        i = L - 1
        pages = block_table[b]
        p1 = torch.arange(max(0, i - w1 + 1), L, device=q.device)
        p2 = torch.arange(max(0, i - w2 + 1), L, device=q.device)
        take = lambda t, pos: t[cache.rows(pages, pos)].view(-1, cache.hkv, D).float().repeat_interleave(g, 1)
        k1, v1, k2, v2 = take(cache.k1, p1), take(cache.v1, p1), take(cache.k2, p2), take(cache.v2, p2)
        s = torch.einsum("hd,ahd,chd->hac", q[b].float(), k1, k2) * scale
        p = s.flatten(1).softmax(-1).view_as(s)
        out[b] = torch.einsum("hac,ahd,chd->hd", p, v1, v2)
    return out


def simplicial_decode(q, cache: PagedSimplicialCache, block_table, seq_lens, w1: int, w2: int, scale=None):
    """q [B, Hq, D] (bf16 on CUDA); block_table [B, max_pages] int32; seq_lens [B] int32 (including the new
    token, already written to the caches).  Returns [B, Hq, D] in q's dtype."""
    B, Hq, D = q.shape
    g = Hq // cache.hkv
    ok = (q.is_cuda and q.dtype == torch.bfloat16 and D == 128 and w1 in (8, 16, 32) and g * w1 <= 128 and w2 >= w1
          and native.available())
    if not ok:
        return simplicial_decode_reference(q, cache, block_table, seq_lens, w1, w2, scale).to(q.dtype)
    q2 = q.reshape(B, Hq * D).contiguous()
    out = torch.empty_like(q2)
    lse2 = torch.empty(B, Hq, dtype=torch.float32, device=q.device)
    bt, sl = block_table.int().contiguous(), seq_lens.int().contiguous()
    rc = native.lib().nga_simplicial_decode(
        q2.data_ptr(), cache.k1.data_ptr(), cache.k2.data_ptr(), cache.v1.data_ptr(), cache.v2.data_ptr(), out.data_ptr(),
        lse2.data_ptr(), bt.data_ptr(), sl.data_ptr(), q2.stride(0), cache.k1.stride(0), out.stride(0), B, Hq, cache.hkv, D, w1, w2,
        bt.size(1), cache.num_pages, 1.0 / math.sqrt(D) if scale is None else float(scale),
        native.status_word(q.device).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_simplicial_decode")
    return out.view(B, Hq, D)
