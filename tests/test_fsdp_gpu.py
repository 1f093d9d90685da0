"""Fused weight-gather GEMMs of fully-sharded linears (forward: output tiles follow the arrival of the
shards; data gradient: k-blocks follow it) against gather + fp32 matmul.  Child processes, one per GPU."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from archlab_b200.ops import native
    from archlab_b200.parallel.fsdp import FsdpGroup, FsdpLinear

    dev = torch.device("cuda", rank)
    res = {}
    # the three backward policies: second gather by NCCL, second gather inside the data-gradient GEMM, gathered
    # weights kept from the forward pass
    for tag, kw in (("a", {}), ("b", {"fused_dgrad": True}), ("c", {"reshard_after_forward": False})):
        _check_group(FsdpGroup(dev, copy_clusters=2, **kw), tag, res, rank, world, dev)
    torch.cuda.synchronize()
    native.check_status()
    torch.save(res, os.path.join(out_dir, f"fsdp_rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _check_group(grp, tag, res, rank, world, dev):
    import torch.distributed as dist

    from archlab_b200.parallel.fsdp import FsdpLinear

    shapes = [(320, 1024), (1024, 320), (256, 700)]                  # (in, out); 700 pads to 1024 with 2 ranks
    layers = [FsdpLinear(grp, i, o) for i, o in shapes]
    grp.materialize()
    assert grp.fused
    fulls = []
    for n, lay in enumerate(layers):
        g = torch.Generator(device=dev).manual_seed(50 + n)            # the same full weight on every rank
        w = (torch.randn(lay.out_features, lay.in_features, device=dev, generator=g) * 0.1).bfloat16()
        lay.load_full(w)
        fulls.append(w)
    grp.sync()
    for it in range(2):                                                # several epochs on the same scratch and flags
        for n, (lay, w) in enumerate(zip(layers, fulls)):
            g = torch.Generator(device=dev).manual_seed(1000 * it + 10 * n + rank)
            x = (torch.randn(3, 200, lay.in_features, device=dev, generator=g) * 0.5).bfloat16().requires_grad_(True)
            dy = (torch.randn(3, 200, lay.out_features, device=dev, generator=g) * 0.5).bfloat16()
            y = lay(x)
            got_w = grp.gathered_view(lay)[: lay.out_features].clone()
            y.backward(dy)
            xf, wf = x.detach().float(), w.float()
            res[f"y{tag}{it}_{n}"] = _rel(y, xf @ wf.t())
            res[f"dx{tag}{it}_{n}"] = _rel(x.grad, dy.float() @ wf)
            res[f"w{tag}{it}_{n}"] = float((got_w.float() - wf).abs().max())
            dw = dy.float().flatten(0, 1).t() @ xf.flatten(0, 1)       # this rank's full weight gradient
            dist.all_reduce(dw)
            dw /= world
            r0 = rank * lay.rows_per_rank
            nrows = max(0, min(lay.out_features, r0 + lay.rows_per_rank) - r0)
            res[f"dw{tag}{it}_{n}"] = _rel(lay.weight.grad[:nrows], dw[r0: r0 + nrows])
            res[f"pad{tag}{it}_{n}"] = float(lay.weight.grad[nrows:].float().abs().max()) if nrows < lay.rows_per_rank else 0.0
            lay.weight.grad = None


@pytest.mark.parametrize("world", [pytest.param(w, marks=pytest.mark.skipif(torch.cuda.device_count() < w, reason=f"needs {w} GPUs"))
                                   for w in (2, 4, 8)])
def test_fused_weight_gather_gemms(tmp_path, world):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, 29661 + world, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    from conftest import join_ranks

    join_ranks(procs, timeout=300)
    for r in range(world):
        res = torch.load(tmp_path / f"fsdp_rank{r}.pt")
        for k, v in res.items():
            tol = 1e-6 if k.startswith(("w", "pad")) else 1.5e-2
            assert v < tol, (r, k, v)
