"""Benchmark config 1 on CPU: tiny speedrun GPT whose layer 3 is 2-simplicial attention, Muon +
AdamW, two gloo ranks.  The two-rank run (each rank sees half of the global batch, gradients are
averaged inside the distributed optimizer) must reproduce the single-process run of the full batch.
Multi-rank-on-CPU pattern of the reference: tests/test_deepseek_v41_official_moe.py:358-455.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STEPS = 6


def _config():
    from archlab_b200.models.nanochat import GPTConfig
    from archlab_b200.train.speedrun import TrainerConfig

    m = GPTConfig(sequence_len=256, vocab_size=8192, n_layer=4, n_head=4, n_kv_head=4, n_embd=256,
                  simplicial_layers=(3,), simplicial_w1=16, simplicial_w2=64, compute_dtype=torch.float32,
                  matrix_init_recipe="normal-0.02")
    return TrainerConfig(model=m, micro_batch=4, num_iterations=20, embedding_lr=3e-4 / (256 / 768) ** -0.5,
                         seed=0)


def _tokens():
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, 8192, (STEPS, 4, 257), generator=g, dtype=torch.int64)


def _worker(rank, world, init_file, out_dir):
    sys.path.insert(0, ROOT)
    torch.set_num_threads(2)
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    from archlab_b200.train.speedrun import Trainer

    tr = Trainer(_config(), device="cpu")
    toks = _tokens()
    per = toks.size(1) // world
    losses = [tr.train_step(toks[s, rank * per:(rank + 1) * per]) for s in range(STEPS)]
    torch.save({"losses": losses, "c_q": tr.model.transformer.h[3].attn.c_q.weight.detach().clone(),
                "wte": tr.model.transformer.wte.weight.detach().clone()}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.slow
def test_two_gloo_ranks_match_single_process(tmp_path):
    torch.set_num_threads(4)
    from archlab_b200.train.speedrun import Trainer

    tr = Trainer(_config(), device="cpu")
    toks = _tokens()
    single = [tr.train_step(toks[s]) for s in range(STEPS)]
    assert single[-1] < single[0]
    ctx = mp.get_context("spawn")
    init_file = tmp_path / "rdzv"
    procs = [ctx.Process(target=_worker, args=(r, 2, str(init_file), str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
        if p.is_alive():
            p.terminate()
            pytest.fail("gloo worker timed out")
        assert p.exitcode == 0
    r0 = torch.load(tmp_path / "rank0.pt")
    r1 = torch.load(tmp_path / "rank1.pt")
    # each rank reports its own half-batch loss; their mean is the full-batch loss
    mean = [(a + b) / 2 for a, b in zip(r0["losses"], r1["losses"])]
    for a, b in zip(mean, single):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (mean, single)
    assert torch.allclose(r0["c_q"], r1["c_q"]) and torch.allclose(r0["wte"], r1["wte"])
    ref_q = tr.model.transformer.h[3].attn.c_q.weight.detach()
    assert ((r0["c_q"] - ref_q).norm() / ref_q.norm()).item() < 5e-3
