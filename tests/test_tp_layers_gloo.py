"""Tensor-parallel SwiGLU MLP under sequence parallelism (gloo, 2 ranks) equals the dense MLP."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from archlab_b200.parallel.tp_layers import TPMLP

        torch.manual_seed(0)
        H, I, rows = 16, 24, 6
        Wg, Wu, Wd = torch.randn(I, H) * 0.3, torch.randn(I, H) * 0.3, torch.randn(H, I) * 0.3
        X = torch.randn(world * rows, H)
        mlp = TPMLP(H, I, None, world)
        Il = I // world
        with torch.no_grad():
            mlp.gate_up.weight.copy_(torch.cat([Wg[rank * Il:(rank + 1) * Il], Wu[rank * Il:(rank + 1) * Il]]))
            mlp.down.weight.copy_(Wd[:, rank * Il:(rank + 1) * Il])
        xs = X[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
        y = mlp(xs)
        y.square().sum().backward()
        Xd = X.clone().requires_grad_(True)
        Wg_, Wu_, Wd_ = (w.clone().requires_grad_(True) for w in (Wg, Wu, Wd))
        yd = (torch.nn.functional.silu(Xd @ Wg_.t()) * (Xd @ Wu_.t())) @ Wd_.t()
        yd.square().sum().backward()
        ok = torch.allclose(y, yd[rank * rows:(rank + 1) * rows], atol=1e-5, rtol=1e-4)
        ok &= torch.allclose(xs.grad, Xd.grad[rank * rows:(rank + 1) * rows], atol=1e-4, rtol=1e-3)
        ok &= torch.allclose(mlp.down.weight.grad, Wd_.grad[:, rank * Il:(rank + 1) * Il], atol=1e-4, rtol=1e-3)
        ok &= torch.allclose(mlp.gate_up.weight.grad[:Il], Wg_.grad[rank * Il:(rank + 1) * Il], atol=1e-4, rtol=1e-3)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.slow
def test_tp_mlp_matches_dense():
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
        assert dict(out) == {0: True, 1: True}
