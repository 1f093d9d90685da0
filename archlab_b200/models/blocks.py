"""Shared building blocks of the model zoo: norms, rotary variants, hyper-connections, gated multi-
stream residuals, hashed n-gram memories.  Everything here is plain PyTorch with fp32 statistics so it
doubles as the CPU oracle of the fused sm_100a kernels in ``ops/``.

Reference semantics: ``GroupRMSNorm`` / ``FourStreamGatedResidual`` / ``PLEHash`` /
``OwnerShardedPLEEmbedding`` (src/archlab/architectures/qwen38_flash_next_full.py:416-488,632-796),
``MHCConnection`` / ``EngramMemory`` (src/archlab/architectures/base.py:397-459,1061-1206),
``hc_split_sinkhorn`` (src/archlab/architectures/deepseek_v41_math.py:14-33).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------
# norms
# ------------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor | None = None, *, eps: float = 1e-6,
             zero_centered: bool = False) -> torch.Tensor:
    """fp32 statistics; ``zero_centered`` scales by ``1 + weight`` (weights initialised to 0).
    bf16 CUDA inputs run the fused forward / backward kernels."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.size(-1) % 8 == 0 and x.size(-1) <= 8192:
        from ..ops import block_ops

        if block_ops.usable(x):
            if weight is None or (weight.dim() == 1 and weight.numel() == x.size(-1)):
                return block_ops.rms_norm(x, weight, eps=eps, zero_centered=zero_centered)
            if weight.dim() == 2 and x.dim() >= 2 and tuple(x.shape[-2:]) == tuple(weight.shape):
                # one gain row per slice of the second-to-last dimension: the grouped form of the kernel
                y = block_ops.rms_norm(x.flatten(-2), weight.reshape(-1), eps=eps, zero_centered=zero_centered,
                                       groups=weight.size(0))
                return y.view(x.shape)
    xf = x.float()
    y = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * ((1.0 + weight.float()) if zero_centered else weight.float())
    return y.to(x.dtype)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, zero_centered: bool = False):
        super().__init__()
        self.eps, self.zero_centered = eps, zero_centered
        self.weight = nn.Parameter(torch.zeros(dim) if zero_centered else torch.ones(dim))

    def forward(self, x):
        return rms_norm(x, self.weight, eps=self.eps, zero_centered=self.zero_centered)


class GroupRMSNorm(nn.Module):
    """Independent RMSNorm of each of ``streams`` slices packed along the last dimension."""

    def __init__(self, hidden: int, streams: int, eps: float = 1e-6, zero_centered: bool = False):
        super().__init__()
        self.hidden, self.streams, self.eps, self.zero_centered = hidden, streams, eps, zero_centered
        init = torch.zeros if zero_centered else torch.ones
        self.weight = nn.Parameter(init(streams * hidden))

    def forward(self, packed: torch.Tensor) -> torch.Tensor:
        if packed.size(-1) != self.streams * self.hidden:
            raise ValueError("invalid packed residual width")
        g = packed.unflatten(-1, (self.streams, self.hidden))
        w = self.weight.unflatten(0, (self.streams, self.hidden))
        return rms_norm(g, w, eps=self.eps, zero_centered=self.zero_centered).flatten(-2)


# ------------------------------------------------------------------------------------------------
# rotary embeddings
# ------------------------------------------------------------------------------------------------
def rope_tables(T: int, rot_dim: int, base: float = 10000.0, device=None, offset: int = 0):
    """cos/sin of shape [T, rot_dim/2] (fp32)."""
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, device=device, dtype=torch.float32) / rot_dim))
    ang = torch.outer(torch.arange(offset, offset + T, device=device, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, style: str = "half",
               rot_dim: int | None = None) -> torch.Tensor:
    """x [B, T, H, D]; rotates the first ``rot_dim`` channels (partial RoPE) and passes the rest.

    ``half``: pairs (i, i + rot/2) (nanochat, Qwen); ``interleaved``: pairs (2i, 2i + 1)."""
    D = x.size(-1)
    r = D if rot_dim is None else rot_dim
    if (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and style in ("half", "interleaved") and r % 2 == 0
            and cos.size(0) == x.size(1)):
        from ..ops import block_ops

        if block_ops.usable(x):
            return block_ops.rope(x, cos, sin, rot_dim=r, interleaved=style == "interleaved")
    xr, xp = x[..., :r].float(), x[..., r:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    if style == "half":
        a, b = xr[..., : r // 2], xr[..., r // 2:]
        out = torch.cat([a * c - b * s, a * s + b * c], -1)
    elif style == "interleaved":
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)
    else:
        raise ValueError(f"unknown rope style {style!r}")
    return torch.cat([out.to(x.dtype), xp], -1)


def so3_chunk_rope(x: torch.Tensor, positions: torch.Tensor, base: float = 10000.0) -> torch.Tensor:
    """``positions`` must broadcast against ``x.shape[:-1]`` (e.g. ``[1, T, 1]`` for ``[B, T, H, D]``).
    Rotates consecutive channel triples about the (1,1,1)/sqrt(3) axis by a per-triple angle
    ``pos * base^(-i/n)``.  Every rotation has determinant 1, so a 3x3 determinant of three vectors
    rotated at the SAME position is unchanged while vectors at different positions pick up a relative
    rotation (the position signal of the determinant simplicial switch;
    src/archlab/architectures/qwen35_switch.py:62-77).  Channels beyond the last full triple pass."""
    D = x.size(-1)
    n = D // 3
    v = x[..., : 3 * n].float().unflatten(-1, (n, 3))
    inv = base ** (-torch.arange(n, device=x.device, dtype=torch.float32) / max(n, 1))
    ang = positions.float()[..., None] * inv              # positions broadcast against x.shape[:-1]
    c, s = ang.cos()[..., None], ang.sin()[..., None]
    mean = v.mean(-1, keepdim=True)                                             # projection on the axis
    cross = (torch.roll(v, -1, -1) - torch.roll(v, 1, -1)) / math.sqrt(3.0)     # axis x v
    rot = v * c + cross * s + mean * (1 - c)
    return torch.cat([rot.flatten(-2).to(x.dtype), x[..., 3 * n:]], -1)


# ------------------------------------------------------------------------------------------------
# hyper-connections
# ------------------------------------------------------------------------------------------------
def sinkhorn_knopp(logits: torch.Tensor, iterations: int = 20, eps: float = 1e-6) -> torch.Tensor:
    """exp(logits - rowmax) alternately row- and column-normalised: a near doubly-stochastic map."""
    m = torch.exp(logits - logits.amax(-1, keepdim=True))
    for _ in range(iterations):
        m = m / m.sum(-1, keepdim=True).clamp_min(eps)
        m = m / m.sum(-2, keepdim=True).clamp_min(eps)
    return m


def hc_split_sinkhorn(mixes: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, streams: int = 4,
                      iterations: int = 20, eps: float = 1e-6):
    """V4.1 hyper-connection coefficients from a ``(streams + 2) * streams`` projection:
    pre = sigmoid + eps, post = 2 sigmoid, comb = softmax rows + eps, one column normalisation, then
    ``iterations - 1`` row/column rounds (each denominator carries + eps)."""
    if streams < 1 or iterations < 1 or eps <= 0:
        raise ValueError("positive stream count, iterations and epsilon are required")
    if mixes.shape[-1] != (streams + 2) * streams:
        raise ValueError("wrong mHC projection width")
    if scale.shape != (3,) or base.shape != (mixes.shape[-1],):
        raise ValueError("wrong mHC scale/base shape")
    if mixes.is_cuda and streams == 4:
        from ..ops import stream_mix

        if stream_mix.hc_coefficients_usable(mixes, streams, iterations):
            return stream_mix.hc_coefficients(mixes, scale, base, iterations, eps)
    dt = torch.float64 if mixes.dtype == torch.float64 else torch.float32
    mixes, scale, base = mixes.to(dt), scale.to(dt), base.to(dt)
    n = streams
    pre = torch.sigmoid(mixes[..., :n] * scale[0] + base[:n]) + eps
    post = 2 * torch.sigmoid(mixes[..., n:2 * n] * scale[1] + base[n:2 * n])
    comb = (mixes[..., 2 * n:] * scale[2] + base[2 * n:]).unflatten(-1, (n, n)).softmax(-1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(iterations - 1):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    return pre, post, comb


class HyperConnection(nn.Module):
    """Manifold-constrained hyper-connection around one sublayer (n residual streams).

    ``prepare(streams)`` -> (branch input, h_post, h_res); ``combine`` mixes the residual streams by
    the Sinkhorn map and writes the branch output into every stream with weight h_post."""

    def __init__(self, hidden: int, streams: int = 4, sinkhorn_iterations: int = 20, init_gate: float = 0.01):
        super().__init__()
        self.n, self.hidden, self.iters, self.init_gate = streams, hidden, sinkhorn_iterations, init_gate
        width = streams * (streams + 2)
        self.mapping_proj = nn.Linear(streams * hidden, width, bias=False)
        self.alpha = nn.Parameter(torch.full((3,), init_gate))
        self.bias = nn.Parameter(torch.zeros(width))
        self.eps = 1e-6

    @torch.no_grad()
    def init_weights(self):
        nn.init.xavier_uniform_(self.mapping_proj.weight)
        self.alpha.fill_(self.init_gate)
        self.bias.zero_()

    def mappings(self, streams: torch.Tensor):
        n = self.n
        flat = streams.flatten(-2).float()
        inv = torch.rsqrt(flat.square().mean(-1, keepdim=True) + self.eps)
        scales = torch.cat([self.alpha[0].expand(n), self.alpha[1].expand(n), self.alpha[2].expand(n * n)])
        m = F.linear(flat, self.mapping_proj.weight.float()) * inv * scales + self.bias
        h_pre = m[..., :n].sigmoid()
        h_post = 2.0 * m[..., n:2 * n].sigmoid()
        h_res = sinkhorn_knopp(m[..., 2 * n:].unflatten(-1, (n, n)), self.iters, self.eps)
        return h_pre, h_post, h_res

    def prepare(self, streams: torch.Tensor):
        h_pre, h_post, h_res = self.mappings(streams)
        branch_in = (streams.float() * h_pre.unsqueeze(-1)).sum(-2)
        return branch_in.to(streams.dtype), h_post, h_res

    def combine(self, streams, branch_out, h_post, h_res):
        mixed = h_res @ streams.float()
        return (mixed + h_post.unsqueeze(-1) * branch_out.float().unsqueeze(-2)).to(streams.dtype)


class GatedStreamResidual(nn.Module):
    """Packed n-stream gated residual: group norm -> low-rank sigmoid mixing weights -> mean over
    streams gives the sublayer input; ``inject`` writes the branch back with 2*sigmoid weights."""

    def __init__(self, hidden: int, streams: int = 4, low_rank: int = 64, eps: float = 1e-6,
                 zero_centered: bool = False, combine: bool = True):
        super().__init__()
        self.hidden, self.streams = hidden, streams
        packed = hidden * streams
        self.norm = GroupRMSNorm(hidden, streams, eps, zero_centered)
        self.mix_down = nn.Linear(packed, low_rank, bias=False)
        self.mix_up = nn.Linear(low_rank, packed, bias=False)
        self.inject_proj = nn.Linear(packed, streams, bias=False) if combine else None

    def forward(self, packed: torch.Tensor):
        z = self.norm(packed)
        w = torch.sigmoid(self.mix_up(F.silu(self.mix_down(z) / self.streams)))
        shape = (self.streams, self.hidden)
        mixed = (w.unflatten(-1, shape) * z.unflatten(-1, shape)).mean(-2)
        if self.inject_proj is None:
            return mixed
        return mixed, packed, 2 * torch.sigmoid(self.inject_proj(z) / self.streams)

    @staticmethod
    def inject(packed: torch.Tensor, branch: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        return packed + (branch.unsqueeze(-2) * weights.unsqueeze(-1)).flatten(-2)


# ------------------------------------------------------------------------------------------------
# hashed n-gram memories
# ------------------------------------------------------------------------------------------------
def _is_prime(v: int) -> bool:
    if v < 2:
        return False
    if v % 2 == 0:
        return v == 2
    return all(v % d for d in range(3, math.isqrt(v) + 1, 2))


def distinct_prime_sizes(start: int, count: int, divisor: int = 1) -> tuple[int, ...]:
    """``count`` distinct primes >= start whose sum is divisible by ``divisor`` (the last prime is
    advanced until it is) so the concatenated table shards evenly over the optimizer world."""
    sizes, c = [], max(2, int(start))
    while len(sizes) < count:
        if _is_prime(c):
            sizes.append(c)
        c += 1
    while sum(sizes) % divisor:
        c = sizes[-1] + 1
        while not _is_prime(c):
            c += 1
        sizes[-1] = c
    return tuple(sizes)


_M64 = (1 << 64) - 1
_GAMMA, _M1, _M2 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB


def splitmix64(v: int) -> int:
    v = (v + _GAMMA) & _M64
    v = ((v ^ (v >> 30)) * _M1) & _M64
    v = ((v ^ (v >> 27)) * _M2) & _M64
    return (v ^ (v >> 31)) & _M64


def hash_multipliers(vocab: int, ngram: int, *, layer_index: int = 0, seed: int = 1234) -> torch.Tensor:
    """Odd SplitMix64-derived multipliers bounded so token * multiplier fits in int64."""
    half = max(1, (((1 << 63) - 1) // max(vocab, 1)) // 2)
    s0 = seed + 10007 * layer_index
    return torch.tensor([2 * (splitmix64((s0 + _GAMMA * (i + 1)) & _M64) % half) + 1 for i in range(ngram)],
                        dtype=torch.long)


def shift_within_segments(tokens: torch.Tensor, shift: int, eos: int) -> torch.Tensor:
    """tokens[t - shift] when that position lies in the same EOS-delimited segment, else EOS."""
    if shift == 0:
        return tokens
    B, T = tokens.shape
    pos = torch.arange(T, device=tokens.device)
    eos_pos = torch.where(tokens == eos, pos, -1)
    prev = torch.cat([eos_pos.new_full((B, 1), -1), torch.cummax(eos_pos, 1).values[:, :-1]], 1)
    in_seg = pos.unsqueeze(0) - (prev + 1)
    src = pos - shift
    taken = tokens.gather(1, src.clamp_min(0).expand(B, -1))
    ok = (in_seg >= shift) & (src.unsqueeze(0) >= 0)
    return torch.where(ok, taken, torch.full_like(taken, eos))


class NgramHash(nn.Module):
    """Per-layer-embedding n-gram ids: for each order 2..n and each head, xor of multiplier-scaled
    shifted tokens modulo that head's vocabulary, plus the head's row offset."""

    def __init__(self, vocab: int, ngram: int, heads_per_order: int, head_vocab_sizes, eos: int, seed: int = 1234):
        super().__init__()
        self.ngram, self.heads, self.eos = ngram, heads_per_order, eos
        sizes = torch.tensor(list(head_vocab_sizes), dtype=torch.long)
        self.register_buffer("sizes", sizes)
        self.register_buffer("offsets", torch.cat([sizes.new_zeros(1), sizes.cumsum(0)[:-1]]))
        self.register_buffer("multipliers", hash_multipliers(vocab, ngram, seed=seed))

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        tokens = tokens.long()
        sh = [shift_within_segments(tokens, s, self.eos) for s in range(self.ngram)]
        out = []
        for order in range(2, self.ngram + 1):
            lo = (order - 2) * self.heads
            mixed = sh[0] * self.multipliers[0]
            for p in range(1, order):
                mixed = mixed ^ (sh[p] * self.multipliers[p])
            out.append(torch.remainder(mixed.unsqueeze(-1), self.sizes[lo:lo + self.heads]) + self.offsets[lo:lo + self.heads])
        return torch.cat(out, -1)


class _RowsBack(torch.autograd.Function):
    """all_to_all of embedding rows whose backward is the reverse all_to_all."""

    @staticmethod
    def forward(ctx, rows, out_splits, in_splits, group):
        ctx.meta = (out_splits, in_splits, group)
        out = rows.new_empty((sum(out_splits), rows.size(1)))
        dist.all_to_all_single(out, rows.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out_splits, in_splits, group = ctx.meta
        back = g.new_empty((sum(in_splits), g.size(1)))
        dist.all_to_all_single(back, g.contiguous(), in_splits, out_splits, group=group)
        return back, None, None, None


class OwnerShardedEmbedding(nn.Module):
    """A huge hashed table split into ``partitions`` row blocks dealt round-robin to ``owners`` ranks.
    Lookup: ids travel to their owner (all-to-all), rows come back (all-to-all, differentiable)."""

    def __init__(self, partitions: int, rows_per_partition: int, dim: int, *, owner_rank: int = 0, owners: int = 1,
                 group=None):
        super().__init__()
        if partitions % owners or not 0 <= owner_rank < owners:
            raise ValueError("partition count must divide the owner count and the rank must be valid")
        self.partitions, self.rows, self.dim = partitions, rows_per_partition, dim
        self.owner_rank, self.owners, self.group = owner_rank, owners, group
        self.global_partitions = tuple(range(owner_rank, partitions, owners))
        self.tables = nn.ParameterList(nn.Parameter(torch.empty(rows_per_partition * dim)) for _ in self.global_partitions)

    @torch.no_grad()
    def reset_parameters(self, std: float = 0.02):
        for t in self.tables:
            nn.init.normal_(t, std=std)

    def _local(self, enc: torch.Tensor) -> torch.Tensor:
        stacked = torch.stack([t.view(self.rows, self.dim) for t in self.tables])       # [P_local, rows, dim]
        return stacked[torch.div(enc, self.rows, rounding_mode="floor"), torch.remainder(enc, self.rows)]

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        shape = ids.shape
        flat = ids.reshape(-1).long()
        part = torch.div(flat, self.rows, rounding_mode="floor")
        owner = torch.remainder(part, self.owners)
        enc = torch.div(part, self.owners, rounding_mode="floor") * self.rows + torch.remainder(flat, self.rows)
        if self.owners == 1:
            return self._local(enc).view(*shape, self.dim)
        order = owner.argsort(stable=True)
        send = torch.bincount(owner, minlength=self.owners)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        send_l, recv_l = send.tolist(), recv.tolist()
        got = flat.new_empty(sum(recv_l))
        dist.all_to_all_single(got, enc[order].contiguous(), recv_l, send_l, group=self.group)
        rows = _RowsBack.apply(self._local(got), send_l, recv_l, self.group)
        out = torch.empty_like(rows)
        out = out.index_copy(0, order, rows)
        return out.view(*shape, self.dim)


class ShortCausalConv(nn.Module):
    """Depthwise causal conv over normalised inputs, dilated, followed by SiLU; zero-initialised."""

    def __init__(self, hidden: int, kernel: int, dilation: int):
        super().__init__()
        self.kernel, self.dilation = kernel, dilation
        self.weight = nn.Parameter(torch.zeros(hidden, 1, kernel))

    def forward(self, x):
        T = x.size(1)
        y = F.conv1d(rms_norm(x).transpose(1, 2), self.weight.to(x.dtype), padding=(self.kernel - 1) * self.dilation,
                     dilation=self.dilation, groups=x.size(-1))[..., :T]
        return F.silu(y.transpose(1, 2))


class EngramMemory(nn.Module):
    """Suffix n-gram memory: per (order, head) hash table of a distinct prime size; retrieved rows
    are projected to a key (gate: sign-preserving sqrt of the normalised dot with the hidden state)
    and a value; output = gated value + short dilated causal conv of it."""

    def __init__(self, *, hidden: int, memory_dim: int, vocab: int, vocab_multiplier: int = 1, heads: int = 2,
                 orders: tuple[int, ...] = (2, 3), layer_idx: int = 0, seed: int = 0, kernel: int = 4, world: int = 1):
        super().__init__()
        tables = len(orders) * heads
        if memory_dim % tables:
            raise ValueError("Engram memory width must divide evenly across tables")
        self.orders, self.heads, self.hidden = tuple(orders), heads, hidden
        self.max_order = max(orders)
        sizes = distinct_prime_sizes(vocab * vocab_multiplier, tables, divisor=world)
        self.register_buffer("sizes", torch.tensor(sizes), persistent=False)
        self.register_buffer("offsets", torch.tensor([0, *torch.tensor(sizes).cumsum(0)[:-1].tolist()]), persistent=False)
        g = torch.Generator().manual_seed(seed + 10007 * layer_idx)
        self.register_buffer("multipliers", torch.randint(1, 2 ** 31 - 1, (self.max_order,), generator=g) | 1,
                             persistent=False)
        self.embedding = nn.Embedding(sum(sizes), memory_dim // tables)
        self.key_proj = nn.Linear(memory_dim, hidden, bias=False)
        self.value_proj = nn.Linear(memory_dim, hidden, bias=False)
        self.short_conv = ShortCausalConv(hidden, kernel, self.max_order)

    def hash_ids(self, ids: torch.Tensor, pad_id: int) -> torch.Tensor:
        B, T = ids.shape
        sh = [ids] + [torch.cat([ids.new_full((B, d), pad_id), ids[:, : T - d]], 1) for d in range(1, self.max_order)]
        out, t = [], 0
        for order in self.orders:
            mixed = sh[0] * self.multipliers[0]
            for d in range(1, order):
                mixed = mixed ^ (sh[d] * self.multipliers[d])
            for _ in range(self.heads):
                out.append(torch.remainder(mixed, self.sizes[t]) + self.offsets[t])
                t += 1
        return torch.stack(out, -1)

    def forward(self, hidden_states: torch.Tensor, ids: torch.Tensor, pad_id: int) -> torch.Tensor:
        got = self.embedding(self.hash_ids(ids, pad_id)).flatten(-2).to(hidden_states.dtype)
        key, value = self.key_proj(got), self.value_proj(got)
        z = (rms_norm(hidden_states) * rms_norm(key)).sum(-1) / math.sqrt(self.hidden)
        z = z.abs().clamp_min(1e-6).sqrt() * z.sign()
        gated = torch.sigmoid(z).unsqueeze(-1) * value
        return gated + self.short_conv(gated)
