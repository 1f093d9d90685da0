"""Expert-parallel MoE over gloo ranks equals the single-process SparseMoE with the same weights."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from archlab_b200.models import moe


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        full = moe.SparseMoE(16, 24, n_experts=4, top_k=2, n_shared=1, swiglu_limit=7.0)
        full.init_weights(0.3)
        ep = moe.ExpertParallelMoE(16, 24, 4, 2, dist.group.WORLD, swiglu_limit=7.0, n_shared=1)
        le = ep.local_experts
        with torch.no_grad():
            ep.router.copy_(full.router)
            ep.experts.gate_up.copy_(full.experts.gate_up[rank * le:(rank + 1) * le])
            ep.experts.down.copy_(full.experts.down[rank * le:(rank + 1) * le])
            ep.shared.load_state_dict(full.shared.state_dict())
        torch.manual_seed(100 + rank)
        x = torch.randn(2, 7, 16, requires_grad=True)
        y = ep(x)
        y.square().sum().backward()
        x2 = x.detach().clone().requires_grad_(True)
        want = full(x2)
        want.square().sum().backward()
        ok = torch.allclose(y, want, atol=1e-5, rtol=1e-4) and torch.allclose(x.grad, x2.grad, atol=1e-4, rtol=1e-3)
        # local expert grads, summed over ranks' tokens, equal the full model's grads summed over ranks
        g_full = full.experts.down.grad[rank * le:(rank + 1) * le].clone()
        parts = [torch.zeros_like(full.experts.down.grad) for _ in range(world)]
        dist.all_gather(parts, full.experts.down.grad)
        g_sum = sum(parts)[rank * le:(rank + 1) * le]
        ok = ok and torch.allclose(ep.experts.down.grad, g_sum, atol=1e-4, rtol=1e-3)
        out[rank] = bool(ok)
        del g_full
    finally:
        dist.destroy_process_group()


@pytest.mark.slow
def test_expert_parallel_matches_single_process():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
