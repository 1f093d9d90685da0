"""Evaluation in the training loop: bits-per-byte on held-out tokens (tokenizer independent), a
multiple-choice scorer (the CORE-style "lowest mean loss over the continuation" rule) and batched
sampling (src/archlab/speedrun/loss_eval.py:20-64, core_eval.py:160-270, engine.py)."""
from __future__ import annotations

import math
from collections.abc import Iterable

import torch
import torch.distributed as dist
import torch.nn.functional as F


@torch.no_grad()
def evaluate_bpb(model, batches: Iterable[tuple[torch.Tensor, torch.Tensor]], token_bytes: torch.Tensor, *, group=None) -> float:
    """``token_bytes[v]`` = UTF-8 length of token v (0 for special tokens, which are excluded from both sums).
    bpb = sum(nats) / (ln 2 * sum(bytes)), reduced over all ranks."""
    total_nats = torch.zeros((), dtype=torch.float64, device=token_bytes.device)
    total_bytes = torch.zeros((), dtype=torch.int64, device=token_bytes.device)
    was_training = model.training
    model.eval()
    for x, y in batches:
        loss = model(x, y, loss_reduction="none") if _takes_reduction(model) else _per_token(model, x, y)
        valid = y >= 0
        nbytes = torch.where(valid, token_bytes[y.clamp_min(0)], torch.zeros_like(y))
        counted = nbytes > 0
        total_nats += (loss.double().reshape(y.shape) * counted).sum()
        total_bytes += nbytes.sum()
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(total_nats, group=group)
        dist.all_reduce(total_bytes, group=group)
    model.train(was_training)
    return float("inf") if int(total_bytes) == 0 else float(total_nats) / (math.log(2) * int(total_bytes))


def _takes_reduction(model) -> bool:
    import inspect

    return "loss_reduction" in inspect.signature(model.forward).parameters


def _per_token(model, x, y):
    logits = model(x).float()
    return F.cross_entropy(logits.flatten(0, 1), y.flatten(), ignore_index=-1, reduction="none").view_as(y)


@torch.no_grad()
def score_multiple_choice(model, prefix: list[int], continuations: list[list[int]]) -> int:
    """Index of the continuation with the lowest mean token loss given the shared prefix."""
    dev = next(model.parameters()).device
    losses = []
    for cont in continuations:
        ids = torch.tensor([prefix + cont], device=dev)
        lp = _per_token(model, ids[:, :-1], ids[:, 1:])[0, len(prefix) - 1:]
        losses.append(float(lp.mean()))
    return min(range(len(losses)), key=losses.__getitem__)


@torch.no_grad()
def generate_batch(model, prompts: list[list[int]], max_tokens: int, *, temperature: float = 0.0, top_k: int | None = None,
                   seed: int = 0, eos: int | None = None) -> list[list[int]]:
    """Greedy / sampled continuation of several prompts at once (right-aligned, left-padded with the first
    token; the padding never influences a causal model's later positions beyond the prompt itself)."""
    dev = next(model.parameters()).device
    width = max(len(p) for p in prompts)
    ids = torch.tensor([[p[0]] * (width - len(p)) + p for p in prompts], device=dev)
    gen = torch.Generator(device=dev).manual_seed(seed)
    done = torch.zeros(len(prompts), dtype=torch.bool, device=dev)
    outs: list[list[int]] = [[] for _ in prompts]
    for _ in range(max_tokens):
        logits = model(ids)[:, -1, :].float()
        if top_k:
            kth = logits.topk(min(top_k, logits.size(-1))).values[:, -1:]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        nxt = torch.multinomial((logits / temperature).softmax(-1), 1, generator=gen) if temperature > 0 else logits.argmax(-1, keepdim=True)
        for i, t in enumerate(nxt[:, 0].tolist()):
            if not done[i]:
                outs[i].append(t)
        if eos is not None:
            done |= nxt[:, 0] == eos
            if bool(done.all()):
                break
        ids = torch.cat([ids, nxt], 1)
    return outs


# ---- task suite and prompt sets of the training loop -----------------------------------------------------------------
def load_task_bundle(path, tokenizer=None) -> dict[str, dict]:
    """A JSON task bundle: ``{task: {"random_baseline": b, "items": [{"prefix": ..., "choices": [...], "gold": i}, ...]}}``.
    ``prefix`` / ``choices`` are token-id lists, or strings when a tokenizer is given (the prefix is encoded with a
    leading BOS, each choice as the continuation of the prefix text)."""
    import json
    from pathlib import Path

    bundle = json.loads(Path(path).read_text())
    out = {}
    for task, body in bundle.items():
        items = []
        for it in body["items"]:
            prefix, choices = it["prefix"], it["choices"]
            if isinstance(prefix, str):
                if tokenizer is None:
                    raise ValueError(f"task {task} holds text; a tokenizer is needed")
                base = tokenizer.encode(prefix, prepend_bos=True)
                choices = [tokenizer.encode(prefix + c, prepend_bos=True)[len(base):] for c in choices]
                prefix = base
            if not 0 <= int(it["gold"]) < len(choices) or any(len(c) == 0 for c in choices) or len(prefix) == 0:
                raise ValueError(f"malformed item in task {task}")
            items.append({"prefix": list(prefix), "choices": [list(c) for c in choices], "gold": int(it["gold"])})
        if not items or not 0 <= body["random_baseline"] < 1:
            raise ValueError(f"task {task} needs items and a baseline in [0, 1)")
        out[task] = {"random_baseline": float(body["random_baseline"]), "items": items}
    return out


@torch.no_grad()
def evaluate_core(model, tasks: dict[str, dict], *, max_per_task: int = -1, rank: int = 0, world: int = 1, group=None) -> dict:
    """Accuracy per task (items strided over the ranks, counts all-reduced), centred accuracies and their mean."""
    from ..data.tokenizer import core_metric

    dev = next(model.parameters()).device
    was_training = model.training
    model.eval()
    acc = {}
    for task, body in tasks.items():
        items = body["items"][:max_per_task] if max_per_task > 0 else body["items"]
        hits = torch.zeros(2, dtype=torch.float64, device=dev)
        for it in items[rank::world]:
            hits[0] += score_multiple_choice(model, it["prefix"], it["choices"]) == it["gold"]
            hits[1] += 1
        if world > 1:
            dist.all_reduce(hits, group=group)
        acc[task] = float(hits[0] / hits[1].clamp_min(1))
    model.train(was_training)
    base = {t: tasks[t]["random_baseline"] for t in tasks}
    centered = {t: (acc[t] - base[t]) / (1.0 - base[t]) for t in tasks}
    return {"results": acc, "centered_results": centered, "core_metric": core_metric(acc, base)}


def load_prompts(path, tokenizer=None) -> list[list[int]]:
    """A YAML or JSON list of prompts: strings (encoded with a leading BOS) or token-id lists."""
    from pathlib import Path

    import yaml

    doc = yaml.safe_load(Path(path).read_text())
    if isinstance(doc, dict) and "schema_version" in doc:              # a versioned prompt set: rows with id / text / tags
        from ..contracts.prompts import load_prompt_set

        doc = [p.text for p in load_prompt_set(path)]
    prompts = doc.get("prompts") if isinstance(doc, dict) else doc
    if not isinstance(prompts, list) or not prompts:
        raise ValueError("the prompt file holds no prompts")
    out = []
    for p in prompts:
        if isinstance(p, str):
            if tokenizer is None:
                raise ValueError("text prompts need a tokenizer")
            p = tokenizer.encode(p, prepend_bos=True)
        if not p or not all(isinstance(t, int) for t in p):
            raise ValueError("a prompt must be text or a non-empty list of token ids")
        out.append(list(p))
    return out
