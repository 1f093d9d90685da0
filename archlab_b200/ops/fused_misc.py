"""Launchers of the single-pass model-zoo kernels (``csrc/misc_kernels.cu``) with PyTorch statements
as the CPU path and the test oracle: RMSNorm variants, rotary embedding, router scoring + top-k, causal
depthwise convolution, hashed n-gram ids, FP8 / NVFP4 block quantisers, stochastic bf16 rounding."""
from __future__ import annotations

import ctypes as C

import torch

from . import native

_vp, _i, _ll, _f, _u64 = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong
native.register_signature("nga_rmsnorm", [_vp, _vp, _vp, _ll, _i, _i, _f, _i, _vp])
native.register_signature("nga_rope", [_vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _vp])
native.register_signature("nga_router_topk", [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp])
native.register_signature("nga_causal_conv1d", [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp])
native.register_signature("nga_ngram_hash", [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _vp])
native.register_signature("nga_fp8_block_quant", [_vp, _vp, _vp, _ll, _i, _i, _vp])
native.register_signature("nga_nvfp4_quant", [_vp, _vp, _vp, _f, _ll, _vp])
native.register_signature("nga_stochastic_bf16", [_vp, _vp, _ll, _u64, _vp])

SCORE_FN = {"softmax": 0, "sigmoid": 1, "sqrt_softplus": 2}


def _p(t):
    return None if t is None else t.data_ptr()


def _cuda_bf16(x):
    return x.is_cuda and x.dtype == torch.bfloat16 and native.available()


def rmsnorm(x, weight=None, *, groups: int = 1, eps: float = 1e-6, zero_centered: bool = False):
    """x [..., groups * width]; each of the ``groups`` slices is normalised on its own."""
    from ..models.blocks import rms_norm

    width = x.size(-1) // groups
    if not _cuda_bf16(x) or width % 8:
        w = None if weight is None else weight.view(groups, width)
        return rms_norm(x.unflatten(-1, (groups, width)), w, eps=eps, zero_centered=zero_centered).flatten(-2)
    x = x.contiguous()
    y = torch.empty_like(x)
    wf = None if weight is None else weight.float().contiguous()
    rc = native.lib().nga_rmsnorm(_p(x), _p(wf), _p(y), x.numel() // x.size(-1), groups, width, eps, int(zero_centered),
                                  native.stream_ptr())
    native.check(rc, "nga_rmsnorm")
    return y


def rope_(x, cos, sin, *, rot_dim=None, interleaved: bool = False):
    """In-place rotary embedding of x [B, T, H, D] (bf16 CUDA) with tables [T, rot/2]."""
    B, T, H, D = x.shape
    rot = D if rot_dim is None else rot_dim
    if not _cuda_bf16(x) or not x.is_contiguous():
        from ..models.blocks import apply_rope

        x.copy_(apply_rope(x, cos, sin, style="interleaved" if interleaved else "half", rot_dim=rot))
        return x
    rc = native.lib().nga_rope(_p(x), _p(cos.float().contiguous()), _p(sin.float().contiguous()), B * T, T, H, D, rot,
                               int(interleaved), native.stream_ptr())
    native.check(rc, "nga_rope")
    return x


def router_topk(x, weight, bias, *, top_k: int, score: str = "sqrt_softplus", route_scale: float = 1.0, renormalize: bool = True,
                return_scores: bool = False):
    """-> (weights [T, k] fp32, indices [T, k] int64[, scores [T, E]])."""
    T, Cdim = x.shape
    E = weight.size(0)
    if not (_cuda_bf16(x) and weight.dtype == torch.bfloat16 and E <= 512 and Cdim % 8 == 0 and top_k <= 32):
        from ..models.moe import route

        w, idx, sc = route(x, weight, bias, top_k=top_k, score=score, route_scale=route_scale, renormalize=renormalize)
        return (w, idx, sc) if return_scores else (w, idx)
    ow = torch.empty(T, top_k, dtype=torch.float32, device=x.device)
    oi = torch.empty(T, top_k, dtype=torch.int32, device=x.device)
    sc = torch.empty(T, E, dtype=torch.float32, device=x.device) if return_scores else None
    bf = None if bias is None else bias.float().contiguous()
    rc = native.lib().nga_router_topk(_p(x.contiguous()), _p(weight.contiguous()), _p(bf), _p(ow), _p(oi), _p(sc), T, Cdim, E, top_k,
                                      SCORE_FN[score], route_scale, int(renormalize), native.stream_ptr())
    native.check(rc, "nga_router_topk")
    return (ow, oi.long(), sc) if return_scores else (ow, oi.long())


def causal_conv1d(x, weight, bias=None, *, activation="silu", dilation: int = 1):
    """x [B, T, C], weight [C, K]."""
    if not _cuda_bf16(x):
        from .delta_rule import causal_conv1d as ref

        return ref(x, weight, bias, activation, dilation)
    B, T, Cc = x.shape
    x = x.contiguous()
    y = torch.empty_like(x)
    bf = None if bias is None else bias.float().contiguous()
    rc = native.lib().nga_causal_conv1d(_p(x), _p(weight.float().contiguous()), _p(bf), _p(y), B, T, Cc, weight.size(1), dilation,
                                        int(activation == "silu"), native.stream_ptr())
    native.check(rc, "nga_causal_conv1d")
    return y


def ngram_hash(tokens, multipliers, sizes, offsets, *, ngram: int, heads_per_order: int, eos: int):
    """tokens [B, T] int64 -> ids [B, T, (ngram - 1) * heads_per_order]; history stops at EOS boundaries."""
    B, T = tokens.shape
    pos = torch.arange(T, device=tokens.device)
    eos_pos = torch.where(tokens == eos, pos, -1)
    prev = torch.cat([eos_pos.new_full((B, 1), -1), torch.cummax(eos_pos, 1).values[:, :-1]], 1)
    seg_start = (prev + 1).int().contiguous()
    if not (tokens.is_cuda and native.available()):
        from ..models.blocks import shift_within_segments

        sh = [shift_within_segments(tokens, s, eos) for s in range(ngram)]
        out = []
        for order in range(2, ngram + 1):
            lo = (order - 2) * heads_per_order
            mixed = sh[0] * multipliers[0]
            for p in range(1, order):
                mixed = mixed ^ (sh[p] * multipliers[p])
            out.append(torch.remainder(mixed.unsqueeze(-1), sizes[lo:lo + heads_per_order]) + offsets[lo:lo + heads_per_order])
        return torch.cat(out, -1)
    H = (ngram - 1) * heads_per_order
    ids = torch.empty(B, T, H, dtype=torch.int64, device=tokens.device)
    rc = native.lib().nga_ngram_hash(_p(tokens.contiguous()), _p(seg_start), _p(multipliers.contiguous()), _p(sizes.contiguous()),
                                     _p(offsets.contiguous()), _p(ids), B, T, ngram, heads_per_order, eos, native.stream_ptr())
    native.check(rc, "nga_ngram_hash")
    return ids


def fp8_block_quantize(x, block: int = 128, *, pow2: bool = True):
    if not _cuda_bf16(x) or block not in (32, 128):
        from .quant import fp8_block_quantize as ref

        return ref(x, block, pow2=pow2)
    x = x.contiguous()
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(*x.shape[:-1], x.size(-1) // block, dtype=torch.float32, device=x.device)
    rc = native.lib().nga_fp8_block_quant(_p(x), _p(q), _p(s), x.numel(), block, int(pow2), native.stream_ptr())
    native.check(rc, "nga_fp8_block_quant")
    return q, s


def nvfp4_quantize(x, tensor_scale=None):
    """-> (values on the e2m1 grid as bf16, e4m3 block scales [..., n / 16], fp32 tensor scale)."""
    if tensor_scale is None:
        tensor_scale = (x.float().abs().amax().clamp_min(1e-12) / (6.0 * 448.0)).reshape(())
    if not _cuda_bf16(x):
        from .quant import nvfp4_quantize as ref

        return ref(x, tensor_scale=tensor_scale)
    x = x.contiguous()
    vals = torch.empty_like(x)
    bs = torch.empty(*x.shape[:-1], x.size(-1) // 16, dtype=torch.float8_e4m3fn, device=x.device)
    rc = native.lib().nga_nvfp4_quant(_p(x), _p(vals), _p(bs), float(tensor_scale), x.numel(), native.stream_ptr())
    native.check(rc, "nga_nvfp4_quant")
    return vals, bs, tensor_scale


def stochastic_bf16(x: torch.Tensor, seed: int) -> torch.Tensor:
    if not (x.is_cuda and native.available()):
        from .quant import stochastic_bfloat16

        return stochastic_bfloat16(x, generator=torch.Generator(device=x.device).manual_seed(seed))
    x = x.contiguous()
    y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    rc = native.lib().nga_stochastic_bf16(_p(x), _p(y), x.numel(), seed & (2 ** 64 - 1), native.stream_ptr())
    native.check(rc, "nga_stochastic_bf16")
    return y
