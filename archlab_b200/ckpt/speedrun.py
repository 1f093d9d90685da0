"""Speedrun checkpoint bundle (src/archlab/speedrun/checkpoint.py:36-167).

Layout of one step in ``checkpoint_dir``::

    model_{step:06d}.pt            rank 0: model state dict
    meta_{step:06d}.json           rank 0: metadata (must contain "step")
    optim_{step:06d}_rank{r}.pt    every rank: its optimizer shard (ZeRO-1 state is sharded)
    rng_{step:06d}_rank{r}.pt      every rank: python / numpy / torch CPU / torch CUDA RNG state

Every file is written to a temporary name and renamed, so a reader never sees a torn file;
``verify_checkpoint_bundle`` rejects a partially published step.
"""
from __future__ import annotations

import json
import os
import random
import re
from pathlib import Path
from typing import Any

import numpy as np
import torch


def _atomic_torch_save(value: Any, path: Path) -> None:
    tmp = path.with_suffix(path.suffix + f".tmp-rank{os.environ.get('RANK', '0')}")
    torch.save(value, tmp)
    tmp.replace(path)


def _atomic_json_save(value: Any, path: Path) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    with tmp.open("w", encoding="utf-8") as f:
        json.dump(value, f, indent=2)
        f.write("\n")
    tmp.replace(path)


def capture_rng_state() -> dict[str, Any]:
    ns = np.random.get_state()
    return {
        "python": random.getstate(),
        "numpy": {"bit_generator": ns[0], "state": torch.from_numpy(ns[1].copy()), "position": ns[2],
                  "has_gauss": ns[3], "cached_gaussian": ns[4]},
        "torch_cpu": torch.get_rng_state(),
        "torch_cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
    }


def restore_rng_state(state: dict[str, Any]) -> None:
    random.setstate(state["python"])
    ns = state["numpy"]
    np.random.set_state((ns["bit_generator"], ns["state"].cpu().numpy(), ns["position"], ns["has_gauss"],
                         ns["cached_gaussian"]))
    torch.set_rng_state(state["torch_cpu"].cpu())
    if state.get("torch_cuda") is not None:
        if not torch.cuda.is_available():
            raise RuntimeError("checkpoint contains a CUDA RNG state but CUDA is unavailable")
        torch.cuda.set_rng_state(state["torch_cuda"].cpu())


def save_checkpoint(checkpoint_dir, step: int, model_data, optimizer_data, meta_data, rank: int = 0,
                    rng_data=None) -> None:
    d = Path(checkpoint_dir)
    d.mkdir(parents=True, exist_ok=True)
    if rank == 0:
        _atomic_torch_save(model_data, d / f"model_{step:06d}.pt")
        _atomic_json_save(meta_data, d / f"meta_{step:06d}.json")
    if optimizer_data is not None:
        _atomic_torch_save(optimizer_data, d / f"optim_{step:06d}_rank{rank:d}.pt")
    if rng_data is not None:
        _atomic_torch_save(rng_data, d / f"rng_{step:06d}_rank{rank:d}.pt")


def verify_checkpoint_bundle(checkpoint_dir, step: int, *, world_size: int, require_optimizer: bool = True,
                             require_rng: bool = False) -> dict[str, Any]:
    if world_size < 1:
        raise ValueError("world_size must be positive")
    d = Path(checkpoint_dir).expanduser().resolve()
    expected = [d / f"model_{step:06d}.pt", d / f"meta_{step:06d}.json"]
    if require_optimizer:
        expected += [d / f"optim_{step:06d}_rank{r:d}.pt" for r in range(world_size)]
    if require_rng:
        expected += [d / f"rng_{step:06d}_rank{r:d}.pt" for r in range(world_size)]
    missing = [str(p) for p in expected if not p.is_file()]
    empty = [str(p) for p in expected if p.is_file() and p.stat().st_size == 0]
    if missing or empty:
        raise RuntimeError(f"incomplete checkpoint step {step}: missing={missing} empty={empty}")
    meta = json.loads((d / f"meta_{step:06d}.json").read_text(encoding="utf-8"))
    if int(meta.get("step", -1)) != step:
        raise RuntimeError(f"checkpoint metadata step mismatch: {meta.get('step')} != {step}")
    return {"step": step, "world_size": world_size, "optimizer_shards": world_size if require_optimizer else 0,
            "rng_shards": world_size if require_rng else 0,
            "files": [{"path": p.name, "bytes": p.stat().st_size} for p in expected]}


def load_checkpoint(checkpoint_dir, step: int, device, load_optimizer: bool = False, rank: int = 0):
    d = Path(checkpoint_dir)
    model = torch.load(d / f"model_{step:06d}.pt", map_location=device)
    optim = torch.load(d / f"optim_{step:06d}_rank{rank:d}.pt", map_location=device) if load_optimizer else None
    meta = json.loads((d / f"meta_{step:06d}.json").read_text(encoding="utf-8"))
    return model, optim, meta


def load_rng_state(checkpoint_dir, step: int, device, rank: int = 0):
    p = Path(checkpoint_dir) / f"rng_{step:06d}_rank{rank:d}.pt"
    return torch.load(p, map_location=device, weights_only=False) if p.is_file() else None


def find_last_step(checkpoint_dir) -> int:
    steps = [int(m.group(1)) for p in Path(checkpoint_dir).glob("model_*.pt")
             if (m := re.fullmatch(r"model_(\d+)\.pt", p.name))]
    if not steps:
        raise FileNotFoundError(f"No checkpoints found in {checkpoint_dir}")
    return max(steps)


def build_model(checkpoint_dir, step: int, device, phase: str = "eval"):
    """Rebuild a speedrun GPT from a bundle: meta ``model_config`` -> module -> strict state load."""
    assert phase in ("train", "eval")
    from ..models.nanochat import GPT, GPTConfig

    state, _, meta = load_checkpoint(checkpoint_dir, step, device)
    state = {k.removeprefix("_orig_mod."): v for k, v in state.items()}
    if torch.device(device).type == "cpu":
        state = {k: v.float() if isinstance(v, torch.Tensor) and v.dtype == torch.bfloat16 else v
                 for k, v in state.items()}
    kw = dict(meta["model_config"])
    if "compute_dtype" in kw and isinstance(kw["compute_dtype"], str):
        kw["compute_dtype"] = getattr(torch, kw["compute_dtype"].removeprefix("torch."))
    if "simplicial_layers" in kw:
        kw["simplicial_layers"] = tuple(kw["simplicial_layers"])
    with torch.device("meta"):
        model = GPT(GPTConfig(**kw))
    model.to_empty(device=device)
    model.init_weights()
    model.load_state_dict(state, strict=True)
    model.train(phase == "train")
    return model, meta
