"""Two-GPU checks (child processes, NCCL bootstrap on 127.0.0.1): the peer-memory fused ZeRO
optimizer must reproduce the NCCL-decomposed one, and both must keep all ranks' weights equal.
Runs only where at least two GPUs are visible."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir, zero_impl):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from archlab_b200.models.nanochat import GPTConfig
    from archlab_b200.ops import native
    from archlab_b200.train.speedrun import Trainer, TrainerConfig

    cfg = GPTConfig(sequence_len=256, vocab_size=2048, n_layer=4, n_head=2, n_kv_head=2, n_embd=256,
                    compute_dtype=torch.bfloat16, matrix_init_recipe="normal-0.02")
    tr = Trainer(TrainerConfig(model=cfg, micro_batch=2, num_iterations=20, head_chunk=256, zero_impl=zero_impl),
                 device=f"cuda:{rank}")
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, 512, (3, 4, 257), generator=g)
    per = toks.size(1) // world
    losses = [tr.train_step(toks[s, rank * per:(rank + 1) * per].contiguous().pin_memory()) for s in range(3)]
    torch.cuda.synchronize()
    native.check_status()
    st = tr.engine.store
    shadows = {str(k): v.shadow.float().cpu() for k, v in st.groups.items()}
    shadows["wte"] = st.table_shadow("wte").float().cpu()
    shadows["lm_head"] = st.table_shadow("lm_head").float().cpu()
    torch.save({"losses": losses, "shadows": shadows}, os.path.join(out_dir, f"{zero_impl}_rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _run(tmp_path, zero_impl, port):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path), zero_impl)) for r in range(2)]
    for p in procs:
        p.start()
    from conftest import join_ranks

    join_ranks(procs)
    return [torch.load(tmp_path / f"{zero_impl}_rank{r}.pt") for r in range(2)]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_zero_matches_nccl_zero(tmp_path):
    nccl = _run(tmp_path, "nccl", 29611)
    peer = _run(tmp_path, "fused", 29612)
    for res in (nccl, peer):
        for k in res[0]["shadows"]:
            assert torch.equal(res[0]["shadows"][k], res[1]["shadows"][k]), f"ranks diverged on {k}"
    for k, a in nccl[0]["shadows"].items():
        b = peer[0]["shadows"][k]
        assert ((a - b).norm() / a.norm().clamp_min(1e-9)).item() < 2e-2, k
    for a, b in zip(nccl[0]["losses"], peer[0]["losses"]):
        assert abs(a - b) < 5e-2
