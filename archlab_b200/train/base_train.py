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
    # horizon, evaluation cadence and artifact policy of the speedrun script (src/archlab/speedrun/base_train.py:466-642)
    ap.add_argument("--target-flops", type=float, default=-1.0, help="derive the step count from a training-FLOP budget (-1: off)")
    ap.add_argument("--exact-global-batch-replay", action=argparse.BooleanOptionalAction, default=False,
                    help="evaluation consumes whole global batches, so any world size sees the same held-out tokens")
    ap.add_argument("--core-metric-every", type=int, default=-1, help="multiple-choice task suite every N steps (-1: off)")
    ap.add_argument("--core-metric-max-per-task", type=int, default=500)
    ap.add_argument("--core-tasks", default=None, help="JSON task bundle for --core-metric-every (see train.evaluation.load_task_bundle)")
    ap.add_argument("--sample-every", type=int, default=-1, help="greedy samples from the prompt set every N steps (-1: off)")
    ap.add_argument("--prompt-file", default=None, help="YAML / JSON prompt set: a list of strings or of token-id lists")
    ap.add_argument("--tokenizer-dir", default=None, help="tokenizer for byte counts, prompts and task text")
    ap.add_argument("--artifact-policy", choices=("metrics_only", "research", "frozen_historical"), default="metrics_only",
                    help="research requires pinned data, an initialization identity and checkpoints")
    ap.add_argument("--data-manifest", default=None, help="content manifest of --data-dir, verified before the first step")
    ap.add_argument("--data-verification", choices=("metadata", "full"), default="metadata")
    ap.add_argument("--precision-recipe", choices=("bf16", "fp8_block", "nvfp4"), default="bf16",
                    help="bf16 runs the fused engine; the block-scaled recipes run the module path on the block-scaled GEMMs")
    ap.add_argument("--device-type", default="", help="cuda | cpu (empty: autodetect)")
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


def _init_distributed(device_type: str = ""):
    use_cuda = torch.cuda.is_available() if not device_type else device_type == "cuda"
    if "RANK" not in os.environ:
        return 0, 1, torch.device("cuda", 0) if use_cuda else torch.device("cpu")
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0))
    if use_cuda:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, dist.get_world_size(), torch.device("cuda", local)
    dist.init_process_group("gloo")
    return rank, dist.get_world_size(), torch.device("cpu")


def check_artifact_policy(a) -> None:
    """``research`` runs must be reproducible from their artifacts: pinned data, a declared initialization, checkpoints."""
    if a.artifact_policy != "research":
        return
    missing = [what for what, ok in (("--data-dir with --data-manifest", bool(a.data_dir and a.data_manifest)),
                                     ("--initialization-hash", bool(a.initialization_hash)),
                                     ("a final checkpoint", a.save_final_checkpoint)) if not ok]
    if missing:
        raise SystemExit("artifact policy 'research' requires " + ", ".join(missing))


def verify_data(a) -> dict | None:
    """Checks --data-dir against --data-manifest before a single token is read; returns the dataset identity."""
    if not a.data_manifest:
        return None
    if not a.data_dir:
        raise SystemExit("--data-manifest needs --data-dir")
    from ..contracts.provenance import verify_dataset_manifest

    return verify_dataset_manifest(a.data_dir, a.data_manifest, mode=a.data_verification)


def horizon(a, model) -> int:
    """Step count: explicit, from a FLOP budget, or from the tokens-per-parameter ratio (in that order)."""
    if a.num_iterations > 0:
        return a.num_iterations
    if a.target_flops > 0:
        return max(1, round(a.target_flops / (model.estimate_flops() * a.total_batch_size)))
    scaling = model.num_scaling_params()
    n_params = scaling["total"] if isinstance(scaling, dict) else int(scaling)
    return max(1, int(a.target_param_data_ratio * n_params) // a.total_batch_size)


class EvalCadence:
    """What the loop does between optimizer steps: validation bits per byte, the task suite, samples."""

    def __init__(self, a, trainer: Trainer, rank: int, world: int, device, log):
        self.a, self.trainer, self.rank, self.world, self.device, self.log = a, trainer, rank, world, device, log
        self.tokenizer = None
        if a.tokenizer_dir:
            from ..data.tokenizer import BPETokenizer

            self.tokenizer = BPETokenizer.load(Path(a.tokenizer_dir))
        vocab = trainer.model.config.vocab_size
        if self.tokenizer is not None:
            table = list(self.tokenizer.token_bytes())[:vocab]
            self.token_bytes = torch.tensor(table + [0] * (vocab - len(table)), dtype=torch.int64, device=device)
        else:
            self.token_bytes = torch.ones(vocab, dtype=torch.int64, device=device)    # no tokenizer: bits per token
        self.tasks = None
        if a.core_metric_every > 0:
            if not a.core_tasks:
                raise SystemExit("--core-metric-every needs --core-tasks")
            if Path(a.core_tasks).is_dir():                                   # published layout: three task types, percent baselines
                from ..evaluation.core_tasks import read_bundle

                if self.tokenizer is None:
                    raise SystemExit("a CORE bundle directory holds text: --core-tasks DIR needs a tokenizer")
                self.tasks = read_bundle(a.core_tasks)
            else:
                from .evaluation import load_task_bundle

                self.tasks = load_task_bundle(a.core_tasks, self.tokenizer)
        self.prompts = None
        if a.sample_every > 0:
            if not a.prompt_file:
                raise SystemExit("--sample-every needs --prompt-file")
            from .evaluation import load_prompts

            self.prompts = load_prompts(a.prompt_file, self.tokenizer)
        self.min_val_bpb, self.val_bpb = float("inf"), None

    def due(self, every: int, step: int, last: bool, *, at_zero: bool) -> bool:
        return every > 0 and (last or (step % every == 0 and (at_zero or step > 0)))

    def eval_steps(self) -> int:
        a = self.a
        if a.exact_global_batch_replay:
            if a.eval_tokens % a.total_batch_size:
                raise ValueError("exact replay requires eval tokens divisible by total batch tokens")
            return a.eval_tokens // a.total_batch_size * (a.total_batch_size // (a.device_batch_size * a.max_seq_len * self.world))
        return a.eval_tokens // (a.device_batch_size * a.max_seq_len * self.world)

    def _val_batches(self, steps: int):
        a = self.a
        if a.data_dir:
            from ..data.fineweb import FineWebBinaryLoader

            loader = FineWebBinaryLoader(a.data_dir, "val", a.device_batch_size, a.max_seq_len, rank=self.rank, world_size=self.world,
                                         device=self.device)
            for _ in range(steps):
                yield next(loader)
        else:                                   # held-out synthetic stream: same law, a seed the training stream never uses
            gen = ZipfTokens(a.vocab_size, a.max_seq_len, a.device_batch_size, seed=a.seed + 7919, rank=self.rank, pin=False)
            for i in range(steps):
                block = gen.block(i).to(self.device)
                yield block[:, :-1], block[:, 1:]

    def run(self, step: int, last: bool, flops_per_token: int) -> None:
        a, model = self.a, self.trainer.model
        if self.due(a.eval_every, step, last, at_zero=True) and a.eval_tokens > 0:
            from .evaluation import evaluate_bpb

            with torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=self.device.type == "cuda"):
                bpb = evaluate_bpb(model, self._val_batches(self.eval_steps()), self.token_bytes)
            if bpb != bpb or bpb in (float("inf"), float("-inf")):
                raise FloatingPointError(f"non-finite validation BPB at step {step}")
            self.val_bpb, self.min_val_bpb = bpb, min(self.min_val_bpb, bpb)
            self._emit({"kind": "validation", "step": step, "tokens": a.total_batch_size * step, "bpb": bpb, "eval_tokens": a.eval_tokens,
                        "total_training_flops": flops_per_token * a.total_batch_size * step})
        if self.tasks is not None and self.due(a.core_metric_every, step, last, at_zero=False):
            if isinstance(self.tasks, list):
                from ..evaluation.core_tasks import evaluate_bundle

                was = model.training
                model.eval()
                res = evaluate_bundle(lambda ids: model(ids), lambda text: self.tokenizer.encode(text, prepend_bos=True), self.tasks,
                                      max_per_task=a.core_metric_max_per_task, rank=self.rank, world=self.world,
                                      device=next(model.parameters()).device, max_tokens=a.max_seq_len)
                model.train(was)
            else:
                from .evaluation import evaluate_core

                res = evaluate_core(model, self.tasks, max_per_task=a.core_metric_max_per_task, rank=self.rank, world=self.world)
            self._emit({"kind": "core", "step": step, "core_metric": res["core_metric"], "centered_results": res["centered_results"]})
        if self.prompts is not None and self.rank == 0 and self.due(a.sample_every, step, last, at_zero=False):
            from .evaluation import generate_batch

            was = model.training
            model.eval()
            outs = generate_batch(model, self.prompts, 16, temperature=0.0, seed=a.seed)
            model.train(was)
            shown = [self.tokenizer.decode(p + o) if self.tokenizer is not None else o for p, o in zip(self.prompts, outs)]
            self._emit({"kind": "samples", "step": step, "samples": shown})

    def _emit(self, row: dict) -> None:
        if self.log is not None:
            self.log.write(json.dumps(row) + "\n")
            self.log.flush()
        if self.rank == 0:
            print(json.dumps({k: v for k, v in row.items() if k != "samples"} if row["kind"] != "samples" else row), flush=True)


def main(argv=None) -> int:
    a = parse_args(argv)
    if a.arch_family not in (None, "nanochat"):
        return run_arm(a)
    rank, world, device = _init_distributed(a.device_type)
    check_artifact_policy(a)
    data_identity = verify_data(a) if rank == 0 or world == 1 else None
    model_cfg = GPTConfig.from_depth(a.depth, sequence_len=a.max_seq_len, vocab_size=a.vocab_size, aspect_ratio=a.aspect_ratio,
                                     head_dim=a.head_dim, window_pattern=a.window_pattern)
    tokens_per_micro = a.device_batch_size * a.max_seq_len * world
    if a.total_batch_size % tokens_per_micro:
        raise SystemExit("total batch must be a multiple of device batch x sequence length x world size")
    accum = a.total_batch_size // tokens_per_micro
    local_batch = a.device_batch_size * accum
    cfg = TrainerConfig(model=model_cfg, micro_batch=a.device_batch_size, num_iterations=max(a.num_iterations, 1), matrix_lr=a.matrix_lr,
                        embedding_lr=a.embedding_lr, unembedding_lr=a.unembedding_lr, scalar_lr=a.scalar_lr, weight_decay=a.weight_decay,
                        warmup_steps=a.warmup_steps, warmdown_ratio=a.warmdown_ratio, final_lr_frac=a.final_lr_frac, seed=a.seed,
                        zero_impl=a.zero_impl, use_engine=a.precision_recipe == "bf16")
    trainer = Trainer(cfg, device=device)
    precision_report = None
    if a.precision_recipe != "bf16":
        from ..ops.blockscaled import convert_linears

        precision_report = convert_linears(trainer.model, a.precision_recipe)
    iters = horizon(a, trainer.model)
    trainer.schedule.num_iterations = iters
    flops_per_token = trainer.model.estimate_flops()
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
        (run_dir / "config.json").write_text(json.dumps({
            "args": vars(a), "world_size": world, "grad_accum_steps": accum, "num_iterations": iters, "flops_per_token": flops_per_token,
            "artifact_policy": a.artifact_policy, "data_identity": data_identity, "precision": precision_report}, indent=2, default=str))
    start, loop_state = 0, {}
    if a.resume_from_step >= 0:
        start, loop_state = resume(trainer, ckpt_dir, a.resume_from_step, rank, world, device)
    if a.data_dir:
        from ..data.fineweb import FineWebBinaryLoader

        loader = FineWebBinaryLoader(a.data_dir, "train", local_batch, a.max_seq_len, rank=rank, world_size=world, device="cpu",
                                     start_batch_index=start)
        next_block = lambda i: loader.next_block().view(1, -1).unfold(1, a.max_seq_len + 1, a.max_seq_len)[0].contiguous()
        data_tag, data_state = "fineweb", loader.state_dict
    else:
        gen = ZipfTokens(a.vocab_size, a.max_seq_len, local_batch, seed=a.seed, rank=rank, pin=device.type == "cuda")
        next_block, data_tag, data_state = gen.block, "synthetic-zipf", (lambda: {"batch_index": trainer.step_index})
    log = open(a.metrics_path or run_dir / f"metrics_rank{rank}.jsonl", "a") if rank == 0 else None
    cadence = EvalCadence(a, trainer, rank, world, device, log)
    cadence.min_val_bpb = loop_state.get("min_val_bpb", cadence.min_val_bpb)
    smooth, total_time = loop_state.get("smooth_train_loss", 0.0), loop_state.get("total_training_time", 0.0)
    stamps, paused = [time.perf_counter()], 0.0
    step = start
    while True:                                   # iters + 1 passes: evaluation and the final checkpoint follow the last update
        last = step == iters
        cadence.run(step, last, flops_per_token)
        due_save = step > start and a.save_every > 0 and step % a.save_every == 0
        if (last and a.save_final_checkpoint) or due_save:
            t_save = time.perf_counter()
            extra = {"artifact_policy": a.artifact_policy, "data_identity": data_identity, "val_bpb": cadence.val_bpb,
                     "dataloader_state_dict": data_state(),
                     "loop_state": {"min_val_bpb": cadence.min_val_bpb, "smooth_train_loss": smooth, "total_training_time": total_time}}
            save(trainer, ckpt_dir, step, rank, model_cfg, a, extra)
            paused += time.perf_counter() - t_save                               # a checkpoint is not a training interval
        if last:
            break
        t0 = time.perf_counter()
        loss = trainer.train_step(next_block(step))
        step += 1
        if a.finite_check_every > 0 and step % a.finite_check_every == 0 and loss != loss:
            raise FloatingPointError(f"non-finite loss at step {step}")          # classified as a numerical failure
        now = time.perf_counter()
        stamps.append(now - paused)
        smooth = 0.9 * smooth + 0.1 * loss
        if step - start > 10:
            total_time += now - t0                                               # the first steps carry one-off set-up cost
        if log is not None and (a.metrics_every <= 1 or step % a.metrics_every == 0 or step == iters):
            log.write(json.dumps({"kind": "train", "step": step, "loss": loss, "smooth_loss": smooth / (1 - 0.9 ** (step - start)),
                                  "tokens_per_second": a.total_batch_size / (now - t0), "total_training_time": total_time,
                                  "total_training_flops": flops_per_token * a.total_batch_size * step, "data": data_tag}) + "\n")
            log.flush()
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


def save(trainer: Trainer, ckpt_dir, step: int, rank: int, model_cfg: GPTConfig, args, extra: dict | None = None) -> None:
    if hasattr(trainer.optimizer, "gather_master"):
        trainer.optimizer.gather_master()                    # full fp32 weights on every rank before the write
    meta = {"step": step, "model_config": {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in asdict(model_cfg).items()},
            "user_config": {k: v for k, v in vars(args).items()}, "world_size": trainer.world, **(extra or {})}
    ckpt.save_checkpoint(ckpt_dir, step, trainer.model.state_dict(), trainer.optimizer.state_dict(), meta, rank=rank,
                         rng_data=ckpt.capture_rng_state())
    if trainer.world > 1:
        dist.barrier()
    if rank == 0:
        ckpt.verify_checkpoint_bundle(ckpt_dir, step, world_size=trainer.world, require_rng=True)


def resume(trainer: Trainer, ckpt_dir, step: int, rank: int, world: int, device) -> tuple[int, dict]:
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
    return step, dict(meta.get("loop_state") or {})


if __name__ == "__main__":
    raise SystemExit(main())
