"""Fused tensor-parallel GEMMs (all-gather -> GEMM, GEMM -> reduce-scatter) over peer memory against
the decomposed NCCL + fp32 matmul oracle.  Child processes, one per GPU; needs two GPUs."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORLDS = [pytest.param(w, marks=pytest.mark.skipif(torch.cuda.device_count() < w, reason=f"needs {w} GPUs")) for w in (2, 4, 8)]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from archlab_b200.ops import native
    from archlab_b200.parallel import tp as T

    dev = torch.device("cuda", rank)
    rows, K, N = 512, 320, 384
    res = {}
    for form, push in (("push", True), ("pull", False)):
        grp = T.TPGroup(rows, max_k=512, max_n=512, device=dev, copy_clusters=2, push=push)
        _check_forms(T, grp, dev, rank, world, rows, K, N, res, form)
    torch.cuda.synchronize()
    native.check_status()
    torch.save(res, os.path.join(out_dir, f"tp_rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _check_forms(T, grp, dev, rank, world, rows, K, N, res, form):
    import torch.distributed as dist

    for it in range(3):                               # several epochs: flags, double buffering, slot reuse
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = (torch.randn(rows, K, device=dev, generator=g) * 0.5).bfloat16()
        gw = torch.Generator(device=dev).manual_seed(7 + it)
        w = (torch.randn(N, K, device=dev, generator=gw) * 0.1).bfloat16()
        y = T.ag_gemm(grp, x, w)
        ref = T.ag_gemm_reference(x, w)
        res[f"{form}_ag{it}"] = ((y.float() - ref.float()).norm() / ref.float().norm()).item()
        wt = w.t().contiguous()                       # [K, N] MN-major operand
        y2 = T.ag_gemm(grp, x, wt, w_mn=True)
        res[f"{form}_ag_mn{it}"] = ((y2.float() - ref.float()).norm() / ref.float().norm()).item()
        gathered = grp.gathered_view(K)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        res[f"gathered_{form}{it}"] = float((gathered.float() - torch.cat(parts).float()).abs().max())   # own rows included
        a = (torch.randn(world * rows, K, device=dev, generator=g) * 0.5).bfloat16()
        resid = (torch.randn(rows, N, device=dev, generator=g)).bfloat16()
        z = T.gemm_rs(grp, a, w, resid=resid)
        zref = T.gemm_rs_reference(a, w, resid=resid)
        res[f"{form}_rs{it}"] = ((z.float() - zref.float()).norm() / zref.float().norm()).item()


@pytest.mark.parametrize("world", WORLDS)
def test_fused_tp_gemms_match_decomposed(tmp_path, world):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, 29631 + world, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    from conftest import join_ranks

    join_ranks(procs)
    for r in range(world):
        res = torch.load(tmp_path / f"tp_rank{r}.pt")
        for k, v in res.items():
            assert v < (1e-6 if k.startswith("gathered") else 1e-2), (r, k, v)


def _mlp_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from archlab_b200.ops import native
    from archlab_b200.parallel import tp as T
    from archlab_b200.parallel.tp_layers import TPMLP

    dev = torch.device("cuda", rank)
    H, I, rows = 256, 512, 256
    grp = T.TPGroup(rows, max_k=512, max_n=512, device=dev, copy_clusters=2)
    torch.manual_seed(0)
    Wg, Wu, Wd = (torch.randn(I, H, device=dev) * 0.05), (torch.randn(I, H, device=dev) * 0.05), (torch.randn(H, I, device=dev) * 0.05)
    X = torch.randn(world * rows, H, device=dev)
    Il = I // world
    fused, plain = TPMLP(H, I, grp, world).to(dev).bfloat16(), TPMLP(H, I, None, world).to(dev)
    with torch.no_grad():
        for m in (fused, plain):
            m.gate_up.weight.copy_(torch.cat([Wg[rank * Il:(rank + 1) * Il], Wu[rank * Il:(rank + 1) * Il]]))
            m.down.weight.copy_(Wd[:, rank * Il:(rank + 1) * Il])
    xs = X[rank * rows:(rank + 1) * rows]
    xa = xs.bfloat16().clone().requires_grad_(True)
    xb = xs.bfloat16().float().clone().requires_grad_(True)
    resid = torch.randn(rows, H, device=dev).bfloat16()
    ya, yb = fused(xa, resid), plain(xb, resid.float())
    go = torch.randn(rows, H, device=dev)
    ya.backward(go.bfloat16())
    yb.backward(go)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()
    res = {"out": rel(ya, yb), "dx": rel(xa.grad, xb.grad), "dgate_up": rel(fused.gate_up.weight.grad, plain.gate_up.weight.grad),
           "ddown": rel(fused.down.weight.grad, plain.down.weight.grad)}
    torch.cuda.synchronize()
    native.check_status()
    torch.save(res, os.path.join(out_dir, f"mlp_rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_mlp_fused_forward_backward(tmp_path):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_mlp_worker, args=(r, 2, 29633, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    from conftest import join_ranks

    join_ranks(procs)
    for r in range(2):
        for k, v in torch.load(tmp_path / f"mlp_rank{r}.pt").items():
            assert v < 2e-2, (r, k, v)
