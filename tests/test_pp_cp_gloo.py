"""Pipeline (1F1B) and context-parallel attention on gloo ranks reproduce the single-process results."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
import torch.nn.functional as F


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _stack():
    torch.manual_seed(3)
    return nn.ModuleList(nn.Linear(8, 8) for _ in range(5))


def _pp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from archlab_b200.parallel.pp import StageLinks, run_1f1b, split_layers

        layers = _stack()
        mine = split_layers(len(layers), world)[rank]
        links = StageLinks(rank, world, rank - 1 if rank else None, rank + 1 if rank + 1 < world else None)
        torch.manual_seed(7)
        mbs = [(torch.randn(4, 8), torch.randn(4, 8)) for _ in range(6)]

        def stage_fn(x, mb):
            h = mb[0] if x is None else x
            for i in mine:
                h = torch.tanh(layers[i](h))
            return F.mse_loss(h, mb[1]) if links.last else h

        loss = run_1f1b(links, stage_fn, mbs, act_shape=(4, 8), act_dtype=torch.float32, device="cpu", loss_scale=1 / 6)
        ref = _stack()
        total = 0
        for x, y in mbs:
            h = x
            for l in ref:
                h = torch.tanh(l(h))
            total = total + F.mse_loss(h, y) / 6
        total.backward()
        ok = all(torch.allclose(layers[i].weight.grad, ref[i].weight.grad, atol=1e-6) for i in mine)
        ok &= all(layers[i].weight.grad is None for i in range(len(layers)) if i not in mine)
        if links.last:
            ok &= bool(torch.allclose(loss, total.detach(), atol=1e-6))
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def _cp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from archlab_b200.parallel import cp

        torch.manual_seed(11)
        B, T, Hq, Hkv, D = 2, 16, 4, 2, 8
        q, k, v = torch.randn(B, T, Hq, D), torch.randn(B, T, Hkv, D), torch.randn(B, T, Hkv, D)
        w = torch.randn(B, T, Hq, D)
        full = [t.clone().requires_grad_(True) for t in (q, k, v)]
        o = cp._prefix_attention(*full, 0)
        (o * w).sum().backward()
        mine = [cp.shard_sequence(t, rank, world).clone().requires_grad_(True) for t in (q, k, v)]
        om = cp.cp_causal_attention(*mine, rank=rank, world=world)
        (om * cp.shard_sequence(w, rank, world)).sum().backward()
        ok = torch.allclose(om, cp.shard_sequence(o.detach(), rank, world), atol=1e-5)
        for a, b in zip(mine, full):
            ok &= torch.allclose(a.grad, cp.shard_sequence(b.grad, rank, world), atol=1e-5)
        ok &= cp.shard_positions(T, rank, world).tolist() == list(range(rank * 4, rank * 4 + 4)) + list(range((3 - rank) * 4, (3 - rank) * 4 + 4))
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_pipeline_1f1b_matches_single_process(world):
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_pp_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert dict(out) == {r: True for r in range(world)}


def test_context_parallel_attention_matches_full():
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_cp_worker, args=(2, _free_port(), out), nprocs=2, join=True)
        assert dict(out) == {0: True, 1: True}


def test_split_layers():
    from archlab_b200.parallel.pp import split_layers

    assert [list(r) for r in split_layers(5, 2)] == [[0, 1, 2], [3, 4]]
    with pytest.raises(ValueError):
        split_layers(2, 3)
