"""Micro-benchmarks of the hand-written sm_100a kernels against the measured roofline.

``python -m archlab_b200.bench_kernels --op gemm|attention|simplicial|trunk [--small]``

Each case is timed with CUDA events on the launching stream after 3 warm-up launches, with a 256 MB
buffer written between timed launches (larger than the 126 MB L2), median of ``--iters``; one JSON
line per case with the achieved TFLOP/s or GB/s and the fraction of the measured peak
(``MEASURED_PEAKS.json`` beside the repository root when present, else the fallback figures).
``--small`` runs one small case per op (inputs a little larger than L2, well under a GB) and is
the workload the ``ncu`` summaries under ``profiles/`` were captured on.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            hbm, tf, src = float(d.get("hbm_gbs", hbm)), float(d.get("bf16_tflops", tf)), "measured"
        except (ValueError, OSError):
            pass
    return hbm, tf, src


class Timer:
    def __init__(self, iters: int):
        self.iters = iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn) -> float:
        for _ in range(3):
            fn()
        ts = []
        for _ in range(self.iters):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]


def _emit(name, ms, *, flops=None, bytes_=None, extra=None):
    hbm, tf, src = _peaks()
    row = {"case": name, "ms": round(ms, 4)}
    if flops is not None:
        row["tflops"] = round(flops / ms / 1e9, 1)
        row[f"of_{src}_bf16_peak"] = round(flops / ms / 1e9 / tf, 3)
    if bytes_ is not None:
        row["gbs"] = round(bytes_ / ms / 1e6, 1)
        row[f"of_{src}_hbm_peak"] = round(bytes_ / ms / 1e6 / hbm, 3)
    if extra:
        row.update(extra)
    print(json.dumps(row), flush=True)


def bench_gemm(t: Timer, small: bool):
    from .ops import gemm as G

    cases = [("nt_fc_fwd", 32768, 5120, 1280, 0, 0), ("nn_fc_dgrad", 32768, 1280, 5120, 0, 1),
             ("tn_fc_wgrad", 5120, 1280, 32768, 1, 1), ("nt_8192", 8192, 8192, 8192, 0, 0),
             ("nn_lm_head_dgrad", 8192, 1280, 65536, 0, 1)]
    if small:
        cases = [("nt_small", 8192, 5120, 1280, 0, 0)]
    for name, M, N, K, a_mn, b_mn in cases:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for impl in ("pair", "single"):
            ms = t(lambda: G.gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out, impl=impl))
            _emit(f"gemm_{name}_{impl}", ms, flops=2.0 * M * N * K, extra={"M": M, "N": N, "K": K})
        if not small:
            at, bt = (a.t() if a_mn else a), (b if b_mn else b.t())
            ms = t(lambda: torch.matmul(at, bt, out=out))
            _emit(f"gemm_{name}_cublas", ms, flops=2.0 * M * N * K)


def bench_fp8(t: Timer, small: bool):
    """8-bit tensor-core GEMM (tensor scales); the roofline fraction is against the bf16 peak (dense fp8 is twice that)."""
    from .ops import fp8

    cases = [("nt_fc_fwd", 32768, 5120, 1280), ("nt_8192", 8192, 8192, 8192), ("nt_dgrad", 32768, 1280, 5120)]
    if small:
        cases = [("nt_small", 8192, 5120, 1280)]
    for name, M, N, K in cases:
        a = torch.randn(M, K, device="cuda").to(fp8.E4M3)
        b = torch.randn(N, K, device="cuda").to(fp8.E4M3)
        ms = t(lambda: fp8.fp8_gemm(a, b, 1.0))
        _emit(f"fp8_gemm_{name}", ms, flops=2.0 * M * N * K, extra={"M": M, "N": N, "K": K})


def bench_blockscaled(t: Timer, small: bool):
    """Block-scaled GEMMs (scale factors in TMEM) and their quantisers; fractions are against the bf16 peak."""
    from .ops import blockscaled as bs

    cases = [("8192", 8192, 8192, 8192), ("fc_fwd", 32768, 5120, 1280), ("dgrad", 32768, 1280, 5120), ("moe_up", 16384, 2816, 2048)]
    if small:
        cases = [("small", 4096, 4096, 4096)]
    for name, M, N, K in cases:
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        qa, qb = bs.quantize_fp8(a, 128), bs.quantize_fp8(b, -128)
        ms = t(lambda: bs.gemm(qa, qb))
        _emit(f"mxfp8_gemm_{name}", ms, flops=2.0 * M * N * K, extra={"M": M, "N": N, "K": K, "scales": "1x128 / 128x128"})
        ms = t(lambda: bs.quantize_fp8(a, 128))
        _emit(f"mxfp8_quant_rows_{name}", ms, bytes_=3.0 * M * K)
        fa, fb = bs.quantize_nvfp4(a), bs.quantize_nvfp4(b, two_d=True)
        ms = t(lambda: bs.gemm(fa, fb))
        _emit(f"nvfp4_gemm_{name}", ms, flops=2.0 * M * N * K, extra={"M": M, "N": N, "K": K})
        amax = a.abs().amax().float()
        ms = t(lambda: bs.quantize_nvfp4(a, hadamard_seed=3, sr_seed=5, amax=amax))
        _emit(f"nvfp4_quant_rht_sr_{name}", ms, bytes_=2.5 * M * K)


def bench_attention(t: Timer, small: bool):
    from .ops import trunk

    cases = [(16, 2048, 10, 10, -1), (16, 2048, 10, 10, 512)] if not small else [(4, 2048, 10, 10, -1)]
    for B, T, Hq, Hkv, window in cases:
        D = 128
        qkv = (torch.randn(B * T, (Hq + 2 * Hkv) * D, device="cuda") * 0.5).bfloat16()
        dout = (torch.randn(B * T, Hq * D, device="cuda") * 0.1).bfloat16()
        span = T if window < 0 else min(T, window + 1)
        pairs = B * Hq * (T * span - (span * (span - 1)) // 2 if window >= 0 else T * (T + 1) // 2)
        out, lse2 = trunk.attn_fwd(qkv, B, T, Hq, Hkv, D, window)
        ms = t(lambda: trunk.attn_fwd(qkv, B, T, Hq, Hkv, D, window))
        _emit(f"attn_fwd_B{B}_T{T}_w{window}", ms, flops=4.0 * D * pairs)
        ms = t(lambda: trunk.attn_bwd(qkv, out, dout, lse2, B, T, Hq, Hkv, D, window))
        _emit(f"attn_bwd_B{B}_T{T}_w{window}", ms, flops=10.0 * D * pairs)


def simplicial_headline(iters: int = 5) -> dict:
    """2-simplicial attention forward + backward at the headline shape (one sequence of 8192, 16 query / 4 KV heads
    of 128, windows 32 x 512): TFLOP/s over the useful (query, short key, long key) triples."""
    from .ops.simplicial_bwd import simplicial_bwd
    from .ops.simplicial_cuda import simplicial_fwd

    B, N, Hq, Hkv, w1, w2, D = 1, 8192, 16, 4, 32, 512, 128
    t = Timer(iters)
    mk = lambda H: (torch.randn(B, N, H, D, device="cuda") * 0.7).bfloat16()
    q, k1, k2, v1, v2 = mk(Hq), mk(Hkv), mk(Hkv), mk(Hkv), mk(Hkv)
    dout = (torch.randn(B, N, Hq, D, device="cuda") * 0.3).bfloat16()
    i = torch.arange(N, dtype=torch.float64)
    triples = float((torch.clamp(i + 1, max=w1) * torch.clamp(i + 1, max=w2)).sum()) * B * Hq
    out, lse2 = simplicial_fwd(q, k1, k2, v1, v2, w1, w2, D ** -0.5)
    ms_f = t(lambda: simplicial_fwd(q, k1, k2, v1, v2, w1, w2, D ** -0.5))
    ms_b = t(lambda: simplicial_bwd(q, k1, k2, v1, v2, out, dout, lse2, w1, w2, D ** -0.5))
    return {"simplicial_fwd_bwd_tflops": round(14.0 * D * triples / (ms_f + ms_b) / 1e9, 1),
            "simplicial_fwd_ms": round(ms_f, 3), "simplicial_bwd_ms": round(ms_b, 3),
            "simplicial_shape": f"N{N} H{Hq}/{Hkv} D{D} windows {w1}x{w2}, bf16, L2 flushed between iterations"}


def bench_simplicial(t: Timer, small: bool):
    from .ops.simplicial_bwd import simplicial_bwd
    from .ops.simplicial_cuda import simplicial_fwd

    cases = [(1, 8192, 16, 4, 32, 512), (1, 8192, 16, 4, 16, 128), (4, 2048, 10, 10, 16, 64)]
    if small:
        cases = [(1, 2048, 8, 2, 32, 512)]
    for B, N, Hq, Hkv, w1, w2 in cases:
        D = 128
        mk = lambda H: (torch.randn(B, N, H, D, device="cuda") * 0.7).bfloat16()
        q, k1, k2, v1, v2 = mk(Hq), mk(Hkv), mk(Hkv), mk(Hkv), mk(Hkv)
        dout = (torch.randn(B, N, Hq, D, device="cuda") * 0.3).bfloat16()
        scale = D ** -0.5
        # valid (query, short key, long key) triples
        i = torch.arange(N, dtype=torch.float64)
        triples = float((torch.clamp(i + 1, max=w1) * torch.clamp(i + 1, max=w2)).sum()) * B * Hq
        out, lse2 = simplicial_fwd(q, k1, k2, v1, v2, w1, w2, scale)
        ms_f = t(lambda: simplicial_fwd(q, k1, k2, v1, v2, w1, w2, scale))
        _emit(f"simplicial_fwd_N{N}_H{Hq}_{w1}x{w2}", ms_f, flops=4.0 * D * triples)
        ms_b = t(lambda: simplicial_bwd(q, k1, k2, v1, v2, out, dout, lse2, w1, w2, scale))
        _emit(f"simplicial_bwd_N{N}_H{Hq}_{w1}x{w2}", ms_b, flops=10.0 * D * triples)
        _emit(f"simplicial_fwd_bwd_N{N}_H{Hq}_{w1}x{w2}", ms_f + ms_b, flops=14.0 * D * triples)


def bench_delta(t: Timer, small: bool):
    """Gated delta rule forward; FLOPs counted as the chunked algorithm's tensor-core products
    (per 64-token chunk and head: gram 2*128*64*128, W/U 2*2*128*64*64, scan 2*128*64*(128+128+64+128))."""
    from .ops import delta_rule as dr

    cases = [(1, 8192, 16), (4, 8192, 16), (8, 2048, 32)] if not small else [(2, 4096, 16)]
    for B, T, H in cases:
        q, k, v = ((torch.randn(B, T, H, 128, device="cuda")).bfloat16() for _ in range(3))
        decay = -torch.rand(B, T, H, device="cuda") * 0.1
        beta = torch.rand(B, T, H, device="cuda")
        ms = t(lambda: dr.gdn_forward_cuda(q, k, v, decay, beta))
        per_chunk = 2 * 128 * 64 * 128 + 4 * 128 * 64 * 64 + 2 * 128 * 64 * (128 + 128 + 64 + 128)
        _emit(f"gdn_fwd_B{B}_T{T}_H{H}", ms, flops=float(per_chunk) * B * H * (T // 64),
              bytes_=B * T * H * 128 * 2 * 4, extra={"tokens_per_s": round(B * T / ms * 1e3)})


def bench_trunk(t: Timer, small: bool):
    from .ops import trunk

    rows, C = (8192, 1280) if small else (32768, 1280)
    x = torch.randn(rows, C, device="cuda").bfloat16()
    x0 = torch.randn(rows, C, device="cuda").bfloat16()
    a = torch.ones(1, device="cuda")
    ms = t(lambda: trunk.mix_norm_fwd(x, x0, a, a))
    _emit("mix_norm_fwd", ms, bytes_=rows * C * 2 * 4)
    V = 65536
    logits = torch.randn(2048 if small else 8192, V, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (logits.size(0),), device="cuda")
    ms = t(lambda: trunk.softcap_ce_(logits, tgt, 1.0))          # in place: logits -> gradient
    _emit("softcap_ce", ms, bytes_=logits.numel() * 2 * 2)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "fp8", "blockscaled", "attention", "simplicial", "trunk", "delta", "all"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    from .ops import native

    t = Timer(a.iters)
    ops = {"gemm": bench_gemm, "fp8": bench_fp8, "blockscaled": bench_blockscaled, "attention": bench_attention, "simplicial": bench_simplicial, "trunk": bench_trunk, "delta": bench_delta}
    for name, fn in ops.items():
        if a.op in (name, "all"):
            fn(t, a.small)
    torch.cuda.synchronize()
    native.check_status()


if __name__ == "__main__":
    main()
