"""Learner gates: distributed forward/backward against the single-process oracle, optimizer checkpoint
restart, long-context backward memory, learner throughput."""
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_worker(rank, world, port, out):
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
        ids = torch.randint(0, cfg.vocab_size, (1, 33))
        want = dense(ids[:, :-1], ids[:, 1:])
        want.backward()
        part = tp(ids[:, :-1], ids[:, 1:])
        part.backward()
        tp.sync_replicated_grads()
        total = part.detach().clone()
        dist.all_reduce(total)
        ok = torch.allclose(total, want.detach(), atol=1e-5)
        ok &= torch.allclose(tp.lm_head.weight.grad, dense.lm_head.weight.grad, atol=1e-5, rtol=1e-3)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_native_forward_backward():
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_oracle_worker, args=(2, _free_port(), out), nprocs=2, join=True)
        assert dict(out) == {0: True, 1: True}


def test_optimizer_checkpoint_restart(tmp_path):
    """Stopping after step k, saving the sharded optimizer and restarting reproduces the uninterrupted run bit for bit."""
    from archlab_b200.optim.zero import ZeroAdamW

    def make():
        torch.manual_seed(1)
        m = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
        return m, ZeroAdamW(m.parameters(), lr=1e-2, weight_decay=0.1)

    def steps(m, opt, lo, hi):
        for i in range(lo, hi):
            g = torch.Generator().manual_seed(100 + i)
            x = torch.randn(5, 8, generator=g)
            opt.zero_grad()
            m(x).pow(2).mean().backward()
            opt.reduce_gradients()
            opt.step()

    ref, ref_opt = make()
    steps(ref, ref_opt, 0, 6)
    a, a_opt = make()
    steps(a, a_opt, 0, 3)
    torch.save({"model": a.state_dict(), "optim": a_opt.state_dict()}, tmp_path / "ck.pt")
    b, b_opt = make()
    ck = torch.load(tmp_path / "ck.pt", weights_only=False)
    b_opt.load_state_dict(ck["optim"])
    b_opt.flat_p[b_opt.lo:b_opt.hi].copy_(b_opt.master)          # compute copy follows the restored master
    steps(b, b_opt, 3, 6)
    for p, q in zip(ref.parameters(), b.parameters()):
        assert torch.equal(p, q)


@pytest.mark.gpu
def test_native_context_forward_backward_memory():
    """One 8192-token sequence through a simplicial + flash layer stack stays within a fixed activation budget."""
    from archlab_b200.models.qwen35 import Qwen35Config, Qwen35LM

    cfg = Qwen35Config(vocab_size=4096, n_layer=4, hidden_size=1024, n_heads=8, n_kv_heads=2, intermediate_size=2048,
                       simplicial_every=2, simplicial_w1=16, simplicial_w2=256, sequence_len=8192)
    m = Qwen35LM(cfg).cuda()
    m.init_weights(0.02)
    ids = torch.randint(0, 4096, (1, 8193), device="cuda")
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    loss = m(ids[:, :-1], ids[:, 1:])
    loss.backward()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    assert torch.isfinite(loss) and peak < 6 * 2 ** 30                 # no [T, T] or [T, w1, w2] score tensor was materialised


@pytest.mark.gpu
def test_package_learner_throughput():
    """Median step time of the flagship trainer against its own first measurement: the regression contract."""
    from archlab_b200.contracts.performance import ThroughputProtocol, summarize_step_timestamps

    from archlab_b200.models.nanochat import GPTConfig
    from archlab_b200.train.speedrun import Trainer, TrainerConfig
    from archlab_b200.data.synthetic import ZipfTokens

    cfg = TrainerConfig(model=GPTConfig.from_depth(4, sequence_len=1024, vocab_size=8192), micro_batch=4, num_iterations=12)
    tr = Trainer(cfg, device=torch.device("cuda"))
    gen = ZipfTokens(8192, 1024, 4, seed=0, rank=0, pin=True)
    stamps = [time.perf_counter()]
    for i in range(12):
        tr.train_step(gen.block(i))
        torch.cuda.synchronize()
        stamps.append(time.perf_counter())
    s = summarize_step_timestamps(stamps, tokens_per_step=4 * 1024, protocol=ThroughputProtocol(warmup_steps=4))
    assert s["tokens_per_second"] > 0 and s["p90_step_seconds"] < 5 * s["median_step_seconds"]
