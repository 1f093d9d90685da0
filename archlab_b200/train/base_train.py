"""Speedrun training entry: ``torchrun -m archlab_b200.train.base_train --depth 20 ...``.

One rank per GPU.  Builds the depth-parameterised nanochat GPT, the fused engine and the ZeRO-1
Muon / AdamW optimizer, streams token blocks (FineWeb ``.bin`` shards, or deterministic Zipf tokens
when no data directory is given), logs one JSON line per step, and writes resumable checkpoint
bundles (model + per-rank optimizer shard + RNG + meta).  Mirrors the lifecycle of the reference's
``archlab.speedrun.base_train`` (src/archlab/speedrun/base_train.py:129-1640: bootstrap -> model ->
optimizer -> resume -> loop -> checkpoint) without its torch.compile / DDP machinery.
"""
from __future__ import annotations

import argparse
import json
import os
import time
from dataclasses import asdict
from pathlib import Path

import torch
import torch.distributed as dist

from ..ckpt import speedrun as ckpt
from ..data.synthetic import ZipfTokens
from ..models.nanochat import GPTConfig
from ..parallel import collectives as coll
from .speedrun import Trainer, TrainerConfig


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description="nanochat speedrun pretraining on sm_100a kernels")
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--max-seq-len", type=int, default=2048)
    ap.add_argument("--vocab-size", type=int, default=65536)
    ap.add_argument("--device-batch-size", type=int, default=16, help="sequences per micro-batch per rank")
    ap.add_argument("--total-batch-size", type=int, default=524288, help="tokens per optimizer step over all ranks")
    ap.add_argument("--num-iterations", type=int, default=-1)
    ap.add_argument("--target-param-data-ratio", type=float, default=10.5)
    ap.add_argument("--matrix-lr", type=float, default=0.02)
    ap.add_argument("--embedding-lr", type=float, default=0.2)
    ap.add_argument("--unembedding-lr", type=float, default=0.004)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--warmup-steps", type=int, default=40)
    ap.add_argument("--warmdown-ratio", type=float, default=0.65)
    ap.add_argument("--zero-impl", default="auto", choices=["auto", "nccl", "fused"])
    ap.add_argument("--data-dir", default=None, help="FineWeb .bin shard directory; synthetic Zipf tokens when absent")
    ap.add_argument("--run-dir", default="runs/speedrun")
    ap.add_argument("--save-every", type=int, default=-1)
    ap.add_argument("--resume-from-step", type=int, default=-1)
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


def _init_distributed():
    if "RANK" not in os.environ:
        return 0, 1, torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, dist.get_world_size(), torch.device("cuda", local)
    dist.init_process_group("gloo")
    return rank, dist.get_world_size(), torch.device("cpu")


def main(argv=None) -> int:
    a = parse_args(argv)
    rank, world, device = _init_distributed()
    model_cfg = GPTConfig.from_depth(a.depth, sequence_len=a.max_seq_len, vocab_size=a.vocab_size)
    tokens_per_micro = a.device_batch_size * a.max_seq_len * world
    if a.total_batch_size % tokens_per_micro:
        raise SystemExit("total batch must be a multiple of device batch x sequence length x world size")
    accum = a.total_batch_size // tokens_per_micro
    local_batch = a.device_batch_size * accum
    probe = Trainer.__new__(Trainer)                       # parameter count decides the horizon
    iters = a.num_iterations
    cfg = TrainerConfig(model=model_cfg, micro_batch=a.device_batch_size, num_iterations=max(iters, 1), matrix_lr=a.matrix_lr,
                        embedding_lr=a.embedding_lr, unembedding_lr=a.unembedding_lr, weight_decay=a.weight_decay,
                        warmup_steps=a.warmup_steps, warmdown_ratio=a.warmdown_ratio, seed=a.seed, zero_impl=a.zero_impl)
    trainer = Trainer(cfg, device=device)
    del probe
    if iters <= 0:
        scaling = trainer.model.num_scaling_params()
        n_params = scaling["total"] if isinstance(scaling, dict) else int(scaling)
        iters = max(1, int(a.target_param_data_ratio * n_params) // a.total_batch_size)
        trainer.schedule.num_iterations = iters
    run_dir = Path(a.run_dir)
    ckpt_dir = run_dir / "checkpoints"
    if rank == 0:
        run_dir.mkdir(parents=True, exist_ok=True)
        (run_dir / "config.json").write_text(json.dumps({"args": vars(a), "world_size": world, "grad_accum_steps": accum,
                                                         "num_iterations": iters}, indent=2, default=str))
    start = 0
    if a.resume_from_step >= 0:
        start = resume(trainer, ckpt_dir, a.resume_from_step, rank, world, device)
    if a.data_dir:
        from ..data.fineweb import FineWebBinaryLoader

        loader = FineWebBinaryLoader(a.data_dir, local_batch, a.max_seq_len, rank=rank, world_size=world)
        loader.seek(start) if hasattr(loader, "seek") else None
        next_block = lambda i: loader.next_batch_tokens() if hasattr(loader, "next_batch_tokens") else loader.block(i)
        data_tag = "fineweb"
    else:
        gen = ZipfTokens(a.vocab_size, a.max_seq_len, local_batch, seed=a.seed, rank=rank, pin=device.type == "cuda")
        next_block = gen.block
        data_tag = "synthetic-zipf"
    log = open(run_dir / f"metrics_rank{rank}.jsonl", "a") if rank == 0 else None
    t_last = time.perf_counter()
    for step in range(start, iters):
        loss = trainer.train_step(next_block(step))
        if log is not None:
            now = time.perf_counter()
            log.write(json.dumps({"step": step + 1, "loss": loss, "tokens_per_second": a.total_batch_size / (now - t_last),
                                  "data": data_tag}) + "\n")
            log.flush()
            t_last = now
        last = step + 1 == iters
        if (a.save_every > 0 and (step + 1) % a.save_every == 0) or last:
            save(trainer, ckpt_dir, step + 1, rank, model_cfg, a)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def save(trainer: Trainer, ckpt_dir, step: int, rank: int, model_cfg: GPTConfig, args) -> None:
    if hasattr(trainer.optimizer, "gather_master"):
        trainer.optimizer.gather_master()                    # full fp32 weights on every rank before the write
    meta = {"step": step, "model_config": {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in asdict(model_cfg).items()},
            "user_config": {k: v for k, v in vars(args).items()}, "world_size": trainer.world}
    ckpt.save_checkpoint(ckpt_dir, step, trainer.model.state_dict(), trainer.optimizer.state_dict(), meta, rank=rank,
                         rng_data=ckpt.capture_rng_state())
    if trainer.world > 1:
        dist.barrier()
    if rank == 0:
        ckpt.verify_checkpoint_bundle(ckpt_dir, step, world_size=trainer.world, require_rng=True)


def resume(trainer: Trainer, ckpt_dir, step: int, rank: int, world: int, device) -> int:
    ckpt.verify_checkpoint_bundle(ckpt_dir, step, world_size=world, require_rng=True)
    state, optim, meta = ckpt.load_checkpoint(ckpt_dir, step, device, load_optimizer=True, rank=rank)
    if int(meta.get("world_size", world)) != world:
        raise RuntimeError("optimizer shards were written by a different world size")
    trainer.model.load_state_dict(state, strict=True)
    if trainer.engine is not None:
        trainer.engine.refresh_shadows()
    if hasattr(trainer.optimizer, "load_state_dict"):
        trainer.optimizer.load_state_dict(optim)
    rng = ckpt.load_rng_state(ckpt_dir, step, "cpu", rank=rank)
    if rng is not None:
        ckpt.restore_rng_state(rng)
    trainer.step_index = step
    return step


if __name__ == "__main__":
    raise SystemExit(main())
