"""Fully-sharded linears on gloo ranks (decomposed gather + matmul path) reproduce the unsharded model:
outputs, input gradients, shard gradients (mean over ranks) and a few optimizer steps."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model():
    torch.manual_seed(11)
    return nn.Sequential(nn.Linear(64, 320, bias=False), nn.Tanh(), nn.Linear(320, 64, bias=False))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from archlab_b200.parallel.fsdp import FsdpGroup, FsdpLinear, shard_linears

        ref = _model()
        model = shard_linears(_model(), FsdpGroup("cpu"), min_features=64)
        layers = [m for m in model.modules() if isinstance(m, FsdpLinear)]
        assert len(layers) == 2 and layers[0].padded_out == 512 and layers[0].rows_per_rank == 256
        opt = torch.optim.SGD(model.parameters(), lr=0.1)
        ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
        errs = []
        for step in range(3):
            torch.manual_seed(100 + step)
            xs = [torch.randn(6, 64) for _ in range(world)]            # one batch per rank
            x = xs[rank].clone().requires_grad_(True)
            y = model(x)
            loss = y.square().mean()
            opt.zero_grad()
            loss.backward()
            # the unsharded model on every rank's batch, gradients averaged
            ropt.zero_grad()
            xr = [t.clone().requires_grad_(True) for t in xs]
            sum(ref(t).square().mean() for t in xr).div(world).backward()
            errs.append((y - ref(xs[rank])).abs().max().item())
            errs.append((x.grad - xr[rank].grad * world).abs().max().item())
            for lay, rl in zip(layers, (ref[0], ref[2])):
                r0 = rank * lay.rows_per_rank
                want = torch.zeros(lay.rows_per_rank, lay.in_features)
                n = max(0, min(lay.out_features, r0 + lay.rows_per_rank) - r0)
                want[:n] = rl.weight.grad[r0: r0 + n]
                errs.append((lay.weight.grad - want).abs().max().item())
            model[0].group.sync()
            opt.step()
            ropt.step()
            model[0].group.sync()
        full = model[0].group.full_weight(layers[0])[:320]
        errs.append((full - ref[0].weight).abs().max().item())
        from archlab_b200.parallel.fsdp import full_state_dict

        state = full_state_dict(model, model[0].group)                 # loads into the unsharded model as is
        fresh = _model()
        fresh.load_state_dict(state)
        errs.append(max((a - b).abs().max().item() for a, b in zip(fresh.parameters(), ref.parameters())))
        torch.save(errs, os.path.join(out, f"fsdp{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_fsdp_linears_match_unsharded_model(tmp_path):
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        if p.is_alive():
            p.terminate()
            pytest.fail("worker timed out")
        assert p.exitcode == 0
    for r in range(2):
        errs = torch.load(tmp_path / f"fsdp{r}.pt")
        assert max(errs) < 1e-5, errs
