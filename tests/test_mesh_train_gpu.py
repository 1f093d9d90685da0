"""Mesh trainer on two GPUs: Qwen3.5-style model under TP=2 + sequence parallelism over the fused
all-gather->GEMM / GEMM->reduce-scatter kernels, with simplicial and flash attention layers."""
import json
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, run_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    from archlab_b200.ops import native
    from archlab_b200.train import mesh_train

    argv = ["--model=qwen35_small", "--tp=2", "--sequence-parallel", "--seq-len=2048", "--global-batch=2", "--steps=8",
            "--lr=1e-3", f"--run-dir={run_dir}"]
    losses = mesh_train.train(mesh_train.parse_args(argv))
    torch.cuda.synchronize()
    native.check_status()
    assert all(l == l for l in losses)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp2_training_loss_falls(tmp_path):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, 29671, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    assert all(p.exitcode == 0 for p in procs)
    rows = [json.loads(l) for l in open(tmp_path / "metrics_rank0.jsonl")]
    assert len(rows) == 8 and rows[-1]["loss"] < rows[0]["loss"] - 0.3
