"""Times the fused tensor-parallel GEMMs against their roofline and their NCCL-decomposed form.

Launch: ``python -m torch.distributed.run --nproc-per-node W --master-addr 127.0.0.1 -m
archlab_b200.parallel.tp_bench [--rows R --k K --cols N] [--fsdp]``.  Rank 0 prints one JSON line per op:
device time (max over ranks, CUDA events, L2 flushed between iterations), achieved TFLOP/s, the
roofline time = max(FLOPs / GEMM peak, NVLink bytes / link bandwidth) and achieved / roofline.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor(sorted(ts)[len(ts) // 2], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--k", type=int, default=2560)
    ap.add_argument("--n", "--cols", dest="n", type=int, default=3072,
                    help="output width (use --cols under torch.distributed.run, whose own options start with --n)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gemm-peak-tflops", type=float, default=1684.0)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--copy-clusters", type=int, default=12)
    ap.add_argument("--fsdp", action="store_true", help="also time the fused weight-gather GEMMs of a sharded linear")
    ap.add_argument("--sweep", type=int, nargs="*", default=[], help="extra copy-cluster counts to time")
    a = ap.parse_args(argv)
    rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from ..ops import gemm as G
    from . import tp as T

    world = dist.get_world_size()
    dev = torch.device("cuda", rank)
    grp = T.TPGroup(a.rows, a.k, max(a.n, a.k), dev, copy_clusters=a.copy_clusters, push=False)      # pull form (copy clusters)
    grp_push = T.TPGroup(a.rows, a.k, max(a.n, a.k), dev)                                             # owner-push / in-kernel reduce
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    M = world * a.rows
    x = torch.randn(a.rows, a.k, device=dev).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev) * 0.02).bfloat16()
    out = torch.empty(M, a.n, device=dev, dtype=torch.bfloat16)
    full = torch.empty(M, a.k, device=dev, dtype=torch.bfloat16)

    def nccl_ag():
        dist.all_gather_into_tensor(full, x)
        G.gemm(full, w, out=out)

    flops = 2.0 * M * a.n * a.k
    link_bytes = (world - 1) * a.rows * a.k * 2
    roof = max(flops / (a.gemm_peak_tflops * 1e12), link_bytes / (a.link_gbs * 1e9)) * 1e3
    rows = []
    extra = [("barrier_only", grp.barrier), ("gemm_only_full_m", lambda: G.gemm(full, w, out=out))]
    for cc in a.sweep:
        def f(cc=cc):
            grp.copy_clusters = cc
            T.ag_gemm(grp, x, w, out=out)
        extra.append((f"ag_gemm_fused_cc{cc}", f))
    for name, fn in extra:
        ms = _time(fn, a.iters, flush)
        rows.append({"op": name, "ms": ms})
    grp.copy_clusters = a.copy_clusters
    for name, fn in (("ag_gemm_push", lambda: T.ag_gemm(grp_push, x, w, out=out)), ("ag_gemm_fused", lambda: T.ag_gemm(grp, x, w, out=out)),
                     ("ag_gemm_nccl", nccl_ag)):
        ms = _time(fn, a.iters, flush)
        rows.append({"op": name, "ms": ms, "tflops": flops / ms / 1e9, "roofline_ms": roof, "of_roofline": roof / ms})
    # row-parallel: local K slice a.k, output width a.k (o-proj / FC2 shape family), reduce-scatter over rows
    act = torch.randn(M, a.n, device=dev).bfloat16()
    w2 = (torch.randn(a.k, a.n, device=dev) * 0.02).bfloat16()
    y = torch.empty(M, a.k, device=dev, dtype=torch.bfloat16)
    ys = torch.empty(a.rows, a.k, device=dev, dtype=torch.bfloat16)

    def nccl_rs():
        G.gemm(act, w2, out=y)
        dist.reduce_scatter_tensor(ys, y)

    flops2 = 2.0 * M * a.k * a.n
    link2 = (world - 1) * a.rows * a.k * 2
    roof2 = max(flops2 / (a.gemm_peak_tflops * 1e12), link2 / (a.link_gbs * 1e9)) * 1e3
    for name, fn in (("gemm_rs_reduce_in_kernel", lambda: T.gemm_rs(grp_push, act, w2, out=ys)),
                     ("gemm_rs_fused", lambda: T.gemm_rs(grp, act, w2, out=ys)), ("gemm_rs_nccl", nccl_rs),
                     ("gemm_only_rs_shape", lambda: G.gemm(act, w2, out=y))):
        ms = _time(fn, a.iters, flush)
        rows.append({"op": name, "ms": ms, "tflops": flops2 / ms / 1e9, "roofline_ms": roof2, "of_roofline": roof2 / ms})
    if a.fsdp:
        # fully-sharded weight [n, k] (row shards on the ranks): forward x W^T and data gradient dy W with the
        # weight gather inside the GEMM kernel, against an NCCL all-gather of the weight followed by the GEMM
        from .fsdp import FsdpGroup, FsdpLinear

        fg = FsdpGroup(dev, copy_clusters=a.copy_clusters, fused_dgrad=True)
        lay = FsdpLinear(fg, a.k, a.n)
        fg.materialize()
        lay.weight.data.normal_(0, 0.02)
        fg.sync()
        xm = torch.randn(M, a.k, device=dev).bfloat16()
        dym = torch.randn(M, lay.padded_out, device=dev).bfloat16()
        wfull = torch.empty(lay.padded_out, a.k, device=dev, dtype=torch.bfloat16)
        yo = torch.empty(M, lay.padded_out, device=dev, dtype=torch.bfloat16)
        dxo = torch.empty(M, a.k, device=dev, dtype=torch.bfloat16)

        flops3 = 2.0 * M * lay.padded_out * a.k
        link3 = (world - 1) * lay.rows_per_rank * a.k * 2
        roof3 = max(flops3 / (a.gemm_peak_tflops * 1e12), link3 / (a.link_gbs * 1e9)) * 1e3

        def nccl_fwd():
            dist.all_gather_into_tensor(wfull, lay.weight.data)
            G.gemm(xm, wfull, out=yo)

        def nccl_dgrad():
            dist.all_gather_into_tensor(wfull, lay.weight.data)
            G.gemm(dym, wfull, b_mn=True, out=dxo)

        for cc in a.sweep:
            fg.copy_clusters = cc
            for name, tr, src in (("fsdp_fwd_fused", False, xm), ("fsdp_dgrad_fused", True, dym)):
                ms = _time(lambda: fg.gemm(src, lay, tr), a.iters, flush)
                rows.append({"op": f"{name}_cc{cc}", "ms": ms, "tflops": flops3 / ms / 1e9})
        fg.copy_clusters = a.copy_clusters
        for name, fn in (("fsdp_fwd_fused", lambda: fg.gemm(xm, lay, False)), ("fsdp_fwd_nccl", nccl_fwd),
                         ("fsdp_dgrad_fused", lambda: fg.gemm(dym, lay, True)), ("fsdp_dgrad_nccl", nccl_dgrad),
                         ("fsdp_gemm_only", lambda: G.gemm(xm, wfull, out=yo))):
            ms = _time(fn, a.iters, flush)
            rows.append({"op": name, "ms": ms, "tflops": flops3 / ms / 1e9, "roofline_ms": roof3, "of_roofline": roof3 / ms})
    if rank == 0:
        for r in rows:
            r.update(world=world, rows_per_rank=a.rows, k=a.k, n=a.n, peaks="measured cuBLAS bf16 burst / peer copy")
            print(json.dumps(r), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
