"""Qwen3.5 under TP=2 + sequence parallelism (gloo) reproduces the dense model's loss and gradients."""
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
        from archlab_b200.models.qwen35 import Qwen35Config, Qwen35LM
        from archlab_b200.models.qwen35_tp import Qwen35TP

        torch.manual_seed(0)
        cfg = Qwen35Config.tiny(n_layer=2, simplicial_every=2, simplicial_w1=2, simplicial_w2=4)
        dense = Qwen35LM(cfg)
        dense.init_weights(0.1)
        tp = Qwen35TP(cfg, None, world=world, rank=rank)
        tp.load_dense(dense)
        ids = torch.randint(0, cfg.vocab_size, (1, 17))
        x, y = ids[:, :-1], ids[:, 1:]
        want = dense(x, y)
        want.backward()
        part = tp(x, y)
        part.backward()
        tp.sync_replicated_grads()
        total = part.detach().clone()
        dist.all_reduce(total)
        ok = torch.allclose(total, want.detach(), atol=1e-5, rtol=1e-4)
        ok &= torch.allclose(tp.embed.weight.grad, dense.embed.weight.grad, atol=1e-5, rtol=1e-3)
        ok &= torch.allclose(tp.layers[0].input_norm.weight.grad, dense.layers[0].input_norm.weight.grad, atol=1e-5, rtol=1e-3)
        ok &= torch.allclose(tp.layers[1].mlp.down.weight.grad, dense.layers[1].down.weight.grad.chunk(world, 1)[rank], atol=1e-5, rtol=1e-3)
        ok &= torch.allclose(tp.layers[1].attn.o.weight.grad, dense.layers[1].attn.o.weight.grad.chunk(world, 1)[rank], atol=1e-5, rtol=1e-3)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.slow
def test_tp_sp_matches_dense():
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
        assert dict(out) == {0: True, 1: True}
