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
    # architecture arms of the frozen campaigns (contracts/campaigns.py): any family other than the fused nanochat
    # engine is built by the model factory and trained by the mesh trainer's sharded AdamW under data parallelism
    ap.add_argument("--arch-family", default=None, help="campaign family (sota_pool, frontier_pool, kimi_kda, engram, ...)")
    ap.add_argument("--aspect-ratio", type=int, default=64)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--window-pattern", default="L")
    ap.add_argument("--per-head-muon", action="store_true")
    ap.add_argument("--arm-lr", type=float, default=3e-4, help="AdamW learning rate of the architecture-arm path")
    ap.add_argument("--scalar-lr", type=float, default=0.5)
    ap.add_argument("--final-lr-frac", type=float, default=0.05)
    ap.add_argument("--eval-every", type=int, default=-1)
    ap.add_argument("--eval-tokens", type=int, default=0)
    ap.add_argument("--finite-check-every", type=int, default=1)
    ap.add_argument("--run", default="dummy", help="tracking run name (dummy: no tracker)")
    ap.add_argument("--model-tag", default=None, help="names the run directory under --run-dir")
    ap.add_argument("--checkpoint-dir", default=None, help="checkpoint bundle directory (default: <run-dir>/checkpoints)")
    ap.add_argument("--metrics-path", default=None, help="per-step JSON lines of rank 0 (default: <run-dir>/metrics_rank0.jsonl)")
    ap.add_argument("--metrics-every", type=int, default=1)
    ap.add_argument("--no-final-checkpoint", dest="save_final_checkpoint", action="store_false")
    ap.add_argument("--save-final-checkpoint", dest="save_final_checkpoint", action="store_true", default=True)
    ap.add_argument("--max-parameters", type=int, default=0, help="refuse a model with more scaling parameters than this")
    ap.add_argument("--max-training-tokens", type=int, default=0, help="refuse a horizon longer than this many tokens")
    ap.add_argument("--initialization-hash", default=None,
                    help="sha256 over the initial weights (contracts.provenance.hash_named_tensors); a mismatch is refused")
    ap.add_argument("--throughput-warmup-steps", type=int, default=10)
    ap.add_argument("--throughput-measurement-steps", type=int, default=0)
    _add_arm_flags(ap)
    return ap.parse_args(argv)


def _arm_knobs() -> dict[str, object]:
    """Every model argument that appears in the campaign tables, with a sample value that fixes its type."""
    from ..contracts import campaigns as C

    knobs: dict[str, object] = {}
    for table in (C.TEN_M_VARIANTS, *[tuple(v.values()) for v in C.FINEWEB_CAMPAIGN_VARIANTS.values()]):
        for arm in table:
            for key, value in arm.model_kwargs().items():
                if key != "arch_family":
                    knobs.setdefault(key, value)
    return knobs


def _add_arm_flags(ap) -> None:
    for key, sample in _arm_knobs().items():
        flag = "--" + key.replace("_", "-")
        if isinstance(sample, bool):
            ap.add_argument(flag, action="store_true", default=None)
        elif isinstance(sample, (tuple, list)):
            ap.add_argument(flag, type=lambda s: tuple(int(v) for v in s.split(",") if v), default=None)
        else:
            ap.add_argument(flag, type=type(sample), default=None)


def arm_model_kwargs(a) -> dict:
    """The campaign-style model arguments named by the command line (geometry + family + the knobs that were given)."""
    kw = {"arch_family": a.arch_family, "depth": a.depth, "aspect_ratio": a.aspect_ratio, "head_dim": a.head_dim,
          "max_seq_len": a.max_seq_len, "vocab_size": a.vocab_size, "window_pattern": a.window_pattern}
    for key in _arm_knobs():
        value = getattr(a, key, None)
        if value is not None:
            kw[key] = value
    return kw


def run_arm(a) -> int:
    """Trains one campaign arm: the model factory builds the family, the mesh trainer steps it (ZeRO-sharded AdamW
    over the data group, run contract, checkpoints, health checks)."""
    from ..models.factory import campaign_arm_config
    from . import mesh_train

    family, cfg = campaign_arm_config(arm_model_kwargs(a))
    if a.total_batch_size % a.max_seq_len:
        raise SystemExit("total batch must be a multiple of the sequence length")
    if a.num_iterations <= 0:
        raise SystemExit("architecture arms take their frozen step count: pass --num-iterations")
    run_dir = Path(a.run_dir) / (a.model_tag or family)
    argv = [f"--model=factory:{family}", f"--seq-len={a.max_seq_len}", f"--global-batch={a.total_batch_size // a.max_seq_len}",
            f"--micro-batch={a.device_batch_size}", f"--steps={a.num_iterations}", f"--lr={a.arm_lr}",
            f"--weight-decay={a.weight_decay}", f"--seed={a.seed}", f"--run-dir={run_dir}"]
    if a.save_every > 0:
        argv.append(f"--save-every={a.save_every}")
    for key, value in cfg.items():
        if key != "sequence_len":
            argv.append(f"--model-set={key}={json.dumps(list(value) if isinstance(value, tuple) else value)}")
    mesh_train.train(mesh_train.parse_args(argv))
    return 0


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
    if a.arch_family not in (None, "nanochat"):
        return run_arm(a)
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
    n_scaling = trainer.model.num_scaling_params()
    n_scaling = n_scaling["total"] if isinstance(n_scaling, dict) else int(n_scaling)
    if a.max_parameters and n_scaling > a.max_parameters:
        raise SystemExit(f"model has {n_scaling} scaling parameters, more than --max-parameters={a.max_parameters}")
    if a.max_training_tokens and iters * a.total_batch_size > a.max_training_tokens:
        raise SystemExit(f"{iters} steps of {a.total_batch_size} tokens exceed --max-training-tokens={a.max_training_tokens}")
    if a.initialization_hash and a.resume_from_step < 0:
        from ..contracts.provenance import hash_named_tensors

        got = hash_named_tensors(trainer.model.state_dict().items())
        if got != a.initialization_hash:
            raise SystemExit(f"initial weights hash to {got}, not to the declared {a.initialization_hash}")
    run_dir = Path(a.run_dir)
    ckpt_dir = Path(a.checkpoint_dir) if a.checkpoint_dir else run_dir / "checkpoints"
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
    log = open(a.metrics_path or run_dir / f"metrics_rank{rank}.jsonl", "a") if rank == 0 else None
    t_last = time.perf_counter()
    stamps, paused = [t_last], 0.0
    for step in range(start, iters):
        loss = trainer.train_step(next_block(step))
        if a.finite_check_every > 0 and (step + 1) % a.finite_check_every == 0 and loss != loss:
            raise FloatingPointError(f"non-finite loss at step {step + 1}")        # classified as a numerical failure
        now = time.perf_counter()
        stamps.append(now - paused)
        if log is not None and (a.metrics_every <= 1 or (step + 1) % a.metrics_every == 0 or step + 1 == iters):
            log.write(json.dumps({"step": step + 1, "loss": loss, "tokens_per_second": a.total_batch_size / (now - t_last),
                                  "data": data_tag}) + "\n")
            log.flush()
        t_last = now
        last = step + 1 == iters
        if (a.save_every > 0 and (step + 1) % a.save_every == 0) or (last and a.save_final_checkpoint):
            save(trainer, ckpt_dir, step + 1, rank, model_cfg, a)
            paused += time.perf_counter() - now                                  # a checkpoint is not a training interval
            t_last = time.perf_counter()
    if rank == 0 and len(stamps) > 1:
        from ..contracts.performance import ThroughputProtocol, summarize_step_timestamps
        from ..contracts.substrate import atomic_write_json

        proto = ThroughputProtocol(warmup_steps=a.throughput_warmup_steps, measurement_steps=a.throughput_measurement_steps)
        atomic_write_json(run_dir / "throughput.json", summarize_step_timestamps(stamps, tokens_per_step=a.total_batch_size,
                                                                                  protocol=proto))
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
