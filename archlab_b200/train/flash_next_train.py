"""Native trainer entry of the Qwen3.8 / Flash-Next family: run contract, resume compatibility, probe run.

    python -m archlab_b200.train.flash_next_train --model-variant tiny --precision bf16 --run-dir RUN [--probe-steps N]

The training itself is the mesh trainer (``train.mesh_train``) on a factory model with the split-row Muon; this
module adds what the reference's native trainers put around it (src/archlab/megatron/qwen38_flash_next_full_train.py:
120-318, 389-420; src/archlab/megatron/qwen38_train.py:38-39, 198-229):

* ``RUN_CONTRACT.json``: what the run *is* - model geometry and parameter count, parallelism, optimizer recipe,
  precision contract, loss normalisation, tokens per step and step budget, data manifest hash, hashes of the
  implementing source files, runtime versions.  Written once; every attempt also leaves ``contracts/attempt-*.json``
  and ``LATEST_CONTRACT.json``.
* resume compatibility: a directory (or an explicit ``--load-dir``) whose contract differs in loss normalisation,
  model geometry, attention grouping or precision recipe is refused with the reason, before any process group forms.
* a probe run (``--probe-steps``): a few steps with gradient hooks on the parameters most likely to be disconnected
  (gates, per-head norms, residual norms); ``PROBE.json`` records for each whether a finite, non-zero gradient arrived.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import platform
import time
from pathlib import Path

import torch

from ..contracts.substrate import atomic_write_json
from ..optim.split_muon import muon_recipe
from .precision_contract import precision_contract

LOSS_NORMALIZATION = "mean over the label tokens of the global batch"
ATTENTION_GROUPING = "query heads grouped by key/value head (GQA), contiguous groups"
VARIANTS = {"tiny": "qwen38_tiny", "quarter": "qwen38_flash_next_quarter", "27b": "qwen38_27b_text", "27b-quarter": "qwen38_27b_quarter_text"}
PRECISION_FLAGS = {"bf16": "bf16", "fp4": "nvfp4"}        # contract name -> mesh trainer flag
PROBE_SUFFIXES = ("q_gate.weight", "q_norm.weight", "k_norm.weight", "output_norm.weight", "residual.norm.weight",
                  "shared_gate.weight", "a_log", "dt_bias")
_SOURCES = ("models/qwen38.py", "train/mesh_train.py", "train/flash_next_train.py", "optim/split_muon.py", "optim/zero.py",
            "ops/blockscaled.py", "ops/delta_rule.py", "data/token_batches.py")


def _sha256(path: Path) -> str | None:
    return hashlib.sha256(path.read_bytes()).hexdigest() if path.is_file() else None


def build_contract(args, model) -> dict:
    here = Path(__file__).resolve().parent.parent
    cfg = model.config
    cfg_dict = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(vars(cfg))
    steps = args.probe_steps or max(1, -(-args.target_train_tokens // (args.global_batch * args.seq_len)))
    manifest = Path(args.data_root) / "DATA_READY.json" if args.data_root else None
    return {
        "format": "archlab-flash-next-run-v1",
        "model": f"Qwen3.8 family, variant {args.model_variant} ({VARIANTS[args.model_variant]}), from-scratch text pretraining",
        "model_config": json.loads(json.dumps(cfg_dict, default=list)),
        "parameter_count": model.num_scaling_params() if hasattr(model, "num_scaling_params") else
        {"total": sum(p.numel() for p in model.parameters())},
        "optimizer_partition": model.optimizer_contract() if hasattr(model, "optimizer_contract") else None,
        "parallelism": {"tensor": 1, "pipeline": 1, "context": 1, "expert": 1, "mode": "dp-only", "data": int(os.environ.get("WORLD_SIZE", "1"))},
        "execution": {"gradient_reduction": "flat-buffer reduce-scatter (AdamW part), one all-reduce per owner (Muon part)",
                      "bounded_checkpoint_staging": True},
        "optimizer": {**muon_recipe(), "peak_lr": args.lr, "muon_lr": args.muon_lr, "weight_decay": args.weight_decay,
                      "gradient_clip": args.grad_clip},
        "checkpointing": {"format": "per-rank torch files + step marker written last", "host_staging": "one local rank per host at a time"},
        "training": {"loss_normalization": LOSS_NORMALIZATION, "attention_grouping": ATTENTION_GROUPING, "seed": args.seed,
                     "sequence_length": args.seq_len, "micro_batch_sequences": args.micro_batch, "global_batch_sequences": args.global_batch,
                     "tokens_per_step": args.global_batch * args.seq_len, "train_steps": steps, "target_tokens": args.target_train_tokens,
                     "probe": bool(args.probe_steps)},
        "data": {"root": str(args.data_root) if args.data_root else "synthetic Zipf(1.1) ids", "manifest_sha256": _sha256(manifest) if manifest else None,
                 "sharding": "data-parallel rank"},
        "precision": precision_contract(args.precision),
        "implementation_sha256": {rel: _sha256(here / rel) for rel in _SOURCES},
        "runtime": {"torch": torch.__version__, "cuda": torch.version.cuda, "python": platform.python_version()},
        "created_at_unix": time.time(),
    }


def validate_resume(previous: dict, current: dict) -> None:
    """Refuses to continue a run under a contract that changes what its numbers mean."""
    def differs(*path):
        a, b = previous, current
        for key in path:
            a, b = (a or {}).get(key), (b or {}).get(key)
        return a != b

    if differs("training", "loss_normalization"):
        raise RuntimeError("loss normalization changed; use a fresh run directory and weights")
    if differs("model_config"):
        raise RuntimeError("model geometry changed; use a fresh run directory and weights")
    if differs("training", "attention_grouping"):
        raise RuntimeError("native attention grouping changed; use a fresh run directory")
    if differs("precision", "precision"):
        raise RuntimeError("precision recipe changed; use a fresh run directory")


def write_contract(run_dir: Path, payload: dict, *, resume: bool, load_dir: Path | None = None) -> None:
    run_dir.mkdir(parents=True, exist_ok=True)
    contract = run_dir / "RUN_CONTRACT.json"
    if contract.exists() and not resume:
        raise RuntimeError("run directory already contains a contract")
    source = (load_dir.parent / "RUN_CONTRACT.json") if load_dir else contract
    if load_dir and not source.is_file():
        raise RuntimeError("explicit checkpoint source lacks a RUN_CONTRACT.json")
    for earlier in dict.fromkeys((contract, source)):
        if earlier.exists():
            validate_resume(json.loads(earlier.read_text()), payload)
    if not contract.exists():
        atomic_write_json(contract, payload)
    (run_dir / "contracts").mkdir(exist_ok=True)
    atomic_write_json(run_dir / "contracts" / f"attempt-{time.time_ns()}.json", payload)
    atomic_write_json(run_dir / "LATEST_CONTRACT.json", payload)


def install_probe_hooks(model) -> dict:
    """Gradient hooks on the parameters named by ``PROBE_SUFFIXES``; returns the live record they fill."""
    record: dict[str, dict] = {}
    for name, p in model.named_parameters():
        if not p.requires_grad or not name.endswith(PROBE_SUFFIXES):
            continue
        record[name] = {"seen": False, "nonfinite": False}

        def hook(grad, key=name):
            state = record[key]
            state["nonfinite"] |= not bool(torch.isfinite(grad).all())
            state["seen"] |= bool(torch.count_nonzero(grad))
            return grad

        p.register_hook(hook)
    return record


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-variant", choices=sorted(VARIANTS), default="tiny")
    ap.add_argument("--precision", choices=sorted(PRECISION_FLAGS), default="bf16")
    ap.add_argument("--run-dir", type=Path, required=True)
    ap.add_argument("--load-dir", type=Path, default=None, help="continue from a checkpoint directory of another run")
    ap.add_argument("--data-root", type=Path, default=None)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--global-batch", type=int, default=8)
    ap.add_argument("--target-train-tokens", type=int, default=1 << 24)
    ap.add_argument("--probe-steps", type=int, default=0)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--muon-lr", type=float, default=0.02)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--grad-clip", type=float, default=1.0)
    ap.add_argument("--optimizer", choices=["muon_split", "adamw"], default="muon_split")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--contract-only", action="store_true", help="write and validate the contract, then stop")
    return ap.parse_args(argv)


def main(argv=None) -> int:
    from ..models.factory import build_model
    from . import mesh_train

    args = parse_args(argv)
    family = VARIANTS[args.model_variant]
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        shape_model = build_model(family, {"sequence_len": args.seq_len}, device="meta", init=False)
        write_contract(args.run_dir, build_contract(args, shape_model), resume=args.resume, load_dir=args.load_dir)
        del shape_model
    if args.contract_only:
        return 0
    contract = json.loads((args.run_dir / "RUN_CONTRACT.json").read_text()) if rank == 0 else None
    steps = args.probe_steps or (contract or {}).get("training", {}).get("train_steps", 1)
    mesh_argv = [f"--model=factory:{family}", f"--seq-len={args.seq_len}", f"--micro-batch={args.micro_batch}",
                 f"--global-batch={args.global_batch}", f"--steps={steps}", f"--lr={args.lr}", f"--muon-lr={args.muon_lr}",
                 f"--weight-decay={args.weight_decay}", f"--grad-clip={args.grad_clip}", f"--optimizer={args.optimizer}",
                 f"--precision={PRECISION_FLAGS[args.precision]}", f"--seed={args.seed}", f"--run-dir={args.run_dir / 'mesh'}",
                 "--bounded-staging", f"--save-every={steps}"] + (["--resume"] if args.resume else [])
    probe = {}
    hooks = {"model": None}

    def on_step(step, loss):
        if args.probe_steps and rank == 0:
            atomic_write_json(args.run_dir / "PROBE.json", {"steps_done": step + 1, "loss": loss, "gradients": probe})

    if args.probe_steps:
        original = mesh_train._Job.__init__

        def patched(self, *a, **k):               # the hooks go on right after the trainer built its model
            original(self, *a, **k)
            probe.update(install_probe_hooks(self.model))
            hooks["model"] = self.model

        mesh_train._Job.__init__ = patched
        try:
            mesh_train.train(mesh_train.parse_args(mesh_argv), on_step=on_step)
        finally:
            mesh_train._Job.__init__ = original
        if rank == 0:
            dead = sorted(n for n, s in probe.items() if not s["seen"] or s["nonfinite"])
            atomic_write_json(args.run_dir / "PROBE.json", {"steps_done": args.probe_steps, "gradients": probe, "disconnected_or_nonfinite": dead,
                                                           "passed": not dead})
            return 0 if not dead else 1
        return 0
    mesh_train.train(mesh_train.parse_args(mesh_argv), on_step=on_step)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
