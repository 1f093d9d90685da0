"""Qualitative sampling from a training checkpoint of a model that has no incremental inference cache.

Gated-delta layers and hashed n-gram memories keep no shared cache contract, so every new token re-runs the whole prefix:
correct for any model whose ``forward(ids)`` returns logits, slow by design, and only meant for looking at what a
checkpoint writes.  Nothing of the optimizer is loaded or touched.  The receipt records the prompts, the sampling
settings, the produced token ids and where the run happened, so two checkpoints can be compared on identical prompts.
(Reference: src/archlab/megatron/qwen38_flash_next_sample.py:1-240.)
"""
from __future__ import annotations

import argparse
import json
import platform
import socket
import time
from pathlib import Path

import torch

from ..contracts.substrate import atomic_write_json
from ..serve.kv_engine import sample_next


@torch.no_grad()
def full_prefix_generate(model, prompt: list[int], *, max_new_tokens: int, temperature: float = 0.0, top_p: float = 1.0, seed: int = 0,
                         stop_tokens: tuple[int, ...] = (), max_context: int | None = None) -> dict:
    if not prompt or max_new_tokens < 1:
        raise ValueError("a non-empty prompt and a positive token budget are required")
    device = next(model.parameters()).device
    rng = torch.Generator(device=device).manual_seed(seed) if temperature > 0 else None
    ids, finish = list(prompt), "length"
    was_training = model.training
    model.eval()
    try:
        for _ in range(max_new_tokens):
            if max_context is not None and len(ids) >= max_context:
                finish = "context"
                break
            logits = model(torch.tensor([ids], dtype=torch.long, device=device))
            logits = logits[0] if isinstance(logits, tuple) else logits
            token = int(sample_next(logits[:, -1].float(), temperature, None, rng, top_p))
            ids.append(token)
            if token in stop_tokens:
                finish = "stop"
                break
    finally:
        model.train(was_training)
    return {"prompt_tokens": len(prompt), "tokens": ids[len(prompt):], "finish_reason": finish}


def sample_prompts(model, prompts: list[list[int]], output, *, checkpoint: str, decode=None, **sampling) -> dict:
    started = time.time()
    rows = []
    base_seed = sampling.pop("seed", 0)
    for i, prompt in enumerate(prompts):
        row = full_prefix_generate(model, prompt, seed=base_seed + i, **sampling)
        if decode is not None:
            row["text"] = decode(row["tokens"])
        rows.append({"index": i, "prompt": prompt, **row})
    receipt = {"format": "archlab-checkpoint-samples-v1", "checkpoint": checkpoint, "sampling": {k: v for k, v in sampling.items() if k != "stop_tokens"},
               "samples": rows, "seconds": time.time() - started, "optimizer_state_loaded": False,
               "environment": {"host": socket.gethostname(), "python": platform.python_version(), "torch": torch.__version__,
                               "device": str(next(model.parameters()).device)}}
    atomic_write_json(Path(output), receipt)
    return receipt


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--factory", required=True, help="module:function that returns the model (weights are loaded from --checkpoint)")
    ap.add_argument("--checkpoint", required=True, help="a state-dict file (torch.save) with the model weights")
    ap.add_argument("--prompts", required=True, help="YAML / JSON prompts (token-id lists, or text with --tokenizer)")
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--output", required=True)
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    a = ap.parse_args(argv)
    import importlib

    from .evaluation import load_prompts

    module, _, function = a.factory.partition(":")
    model = getattr(importlib.import_module(module), function)()
    state = torch.load(a.checkpoint, map_location="cpu", weights_only=True)
    model.load_state_dict(state.get("model", state))
    tokenizer = None
    if a.tokenizer:
        from ..data.tokenizer import BPETokenizer, load_hf

        path = Path(a.tokenizer)
        tokenizer = load_hf(path) if (path / "tokenizer.json").is_file() else BPETokenizer.load(path)
    if torch.cuda.is_available():
        model.cuda()
    receipt = sample_prompts(model, load_prompts(a.prompts, tokenizer), a.output, checkpoint=a.checkpoint, decode=tokenizer.decode if tokenizer else None,
                             max_new_tokens=a.max_new_tokens, temperature=a.temperature, top_p=a.top_p)
    print(json.dumps({"samples": len(receipt["samples"]), "seconds": receipt["seconds"]}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
