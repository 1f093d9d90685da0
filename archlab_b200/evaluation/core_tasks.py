"""The three in-context task types of the CORE suite, from raw items to a correct / incorrect verdict.

* ``multiple_choice``: one prompt per choice (same query, different continuation); the choice with the lowest MEAN token
  loss over its continuation wins.  The continuation span is what follows the COMMON PREFIX of the prompts' tokens.
* ``schema``: one prompt per context option (different context, same continuation); the span is the COMMON SUFFIX; the
  option with the lowest mean loss wins.
* ``language_modeling``: two prompts, without and with the continuation; the item is correct only if the model's argmax
  reproduces EVERY continuation token (exact match), found from the prefix relation of the two token sequences.
Few-shot examples are rendered in front, separated by blank lines; contexts of language-modeling items are trimmed (a
trailing space would merge into the continuation's first token and destroy the prefix relation).  Prompts longer than the
model's context are cropped from the LEFT, with the spans shifted accordingly.
(Reference: src/archlab/speedrun/core_eval.py:19-267.)
"""
from __future__ import annotations

import random
from typing import Callable

import torch
import torch.nn.functional as F

TASK_TYPES = ("multiple_choice", "schema", "language_modeling")


def _shots(examples: list[dict], delimiter: str, kind: str) -> str:
    parts = []
    for ex in examples or []:
        if kind == "multiple_choice":
            parts.append(f"{ex['query']}{delimiter}{ex['choices'][ex['gold']]}")
        elif kind == "schema":
            parts.append(f"{ex['context_options'][ex['gold']]}{delimiter}{ex['continuation']}")
        else:
            parts.append(f"{ex['context'].strip()}{delimiter}{ex['continuation']}")
    return "".join(p + "\n\n" for p in parts)


def render_prompts(item: dict, kind: str, delimiter: str, fewshot: list[dict] | None = None) -> list[str]:
    head = _shots(fewshot, delimiter, kind)
    if kind == "multiple_choice":
        return [f"{head}{item['query']}{delimiter}{choice}" for choice in item["choices"]]
    if kind == "schema":
        return [f"{head}{context}{delimiter}{item['continuation']}" for context in item["context_options"]]
    if kind == "language_modeling":
        without = f"{head}{item['context'].strip()}{delimiter}".strip()
        return [without, f"{head}{item['context'].strip()}{delimiter}{item['continuation']}"]
    raise ValueError(f"unknown task type {kind!r}")


def common_length(sequences: list[list[int]], direction: str = "left") -> int:
    shortest = min(map(len, sequences))
    index = (lambda i: i) if direction == "left" else (lambda i: -1 - i)
    for i in range(shortest):
        token = sequences[0][index(i)]
        if any(s[index(i)] != token for s in sequences):
            return i
    return shortest


def token_spans(kind: str, tokens: list[list[int]]) -> tuple[list[list[int]], list[int], list[int]]:
    """-> (sequences to score, span starts, span ends)."""
    if kind == "multiple_choice":
        start = common_length(tokens, "left")
        return tokens, [start] * len(tokens), [len(t) for t in tokens]
    if kind == "schema":
        tail = common_length(tokens, "right")
        return tokens, [len(t) - tail for t in tokens], [len(t) for t in tokens]
    without, with_ = tokens
    if not len(without) < len(with_) or with_[:len(without)] != without:
        raise ValueError("the prompt without the continuation must be a token prefix of the prompt with it")
    return [with_], [len(without)], [len(with_)]


@torch.no_grad()
def evaluate_item(logits_fn: Callable[[torch.Tensor], torch.Tensor], encode: Callable[[str], list[int]], item: dict, kind: str, *, delimiter: str = " ",
                  fewshot: list[dict] | None = None, max_tokens: int | None = None, pad_id: int = 0, device="cpu") -> bool:
    tokens = [encode(p) for p in render_prompts(item, kind, delimiter, fewshot)]
    sequences, starts, ends = token_spans(kind, tokens)
    if max_tokens is not None:
        cropped = []
        for i, seq in enumerate(sequences):
            cut = max(0, len(seq) - max_tokens)
            cropped.append(seq[cut:])
            starts[i], ends[i] = starts[i] - cut, ends[i] - cut
            if starts[i] < 1:
                raise ValueError("the continuation does not fit the model's context")
        sequences = cropped
    width = max(map(len, sequences))
    ids = torch.full((len(sequences), width), pad_id, dtype=torch.long, device=device)
    for r, seq in enumerate(sequences):
        ids[r, :len(seq)] = torch.tensor(seq, device=device)
    logits = logits_fn(ids).float()
    losses = F.cross_entropy(logits[:, :-1].flatten(0, 1), ids[:, 1:].flatten(), reduction="none").view(len(sequences), width - 1)
    if kind == "language_modeling":
        s, e = starts[0], ends[0]
        return bool(torch.equal(logits[0, s - 1:e - 1].argmax(-1), ids[0, s:e]))
    means = [float(losses[r, starts[r] - 1:ends[r] - 1].mean()) for r in range(len(sequences))]
    return min(range(len(means)), key=means.__getitem__) == item["gold"]


def evaluate_task(logits_fn, encode, data: list[dict], meta: dict, *, rank: int = 0, world: int = 1, seed: int = 1234, **kw) -> tuple[int, int]:
    """(correct, evaluated) over this rank's share of ``data``; few-shot examples are drawn per item with a seed that
    depends on the item index only, never from the item itself."""
    kind, shots = meta["task_type"], int(meta.get("num_fewshot", 0))
    if kind not in TASK_TYPES:
        raise ValueError(f"unknown task type {kind!r}")
    correct = done = 0
    for i in range(rank, len(data), world):
        fewshot = []
        if shots:
            pool = [j for j in range(len(data)) if j != i]
            fewshot = [data[j] for j in random.Random(seed + i).sample(pool, min(shots, len(pool)))]
        correct += int(evaluate_item(logits_fn, encode, data[i], kind, delimiter=meta.get("continuation_delimiter", " "), fewshot=fewshot, **kw))
        done += 1
    return correct, done


def read_bundle(bundle_dir) -> list[dict]:
    """The published bundle layout: ``core.yaml`` (``icl_tasks``: label, icl_task_type, dataset_uri, num_fewshot list,
    optional continuation_delimiter), ``eval_meta_data.csv`` (columns ``Eval Task`` and ``Random baseline`` in PERCENT)
    and ``eval_data/<dataset_uri>`` JSON lines.  A task without a baseline row or a data file fails here, before any
    model time is spent.  (Reference: src/archlab/speedrun/base_eval.py:121-190.)"""
    import csv
    import json
    from pathlib import Path

    import yaml

    root = Path(bundle_dir)
    with open(root / "eval_meta_data.csv", encoding="utf-8", newline="") as f:
        baselines = {row["Eval Task"]: float(row["Random baseline"]) for row in csv.DictReader(f)}
    tasks = []
    for entry in yaml.safe_load((root / "core.yaml").read_text(encoding="utf-8"))["icl_tasks"]:
        label, kind = entry["label"], entry["icl_task_type"]
        if kind not in TASK_TYPES:
            raise ValueError(f"task {label}: unknown task type {kind!r}")
        if label not in baselines or not 0.0 <= baselines[label] < 100.0:
            raise ValueError(f"task {label}: no random baseline in [0, 100) percent")
        path = root / "eval_data" / entry["dataset_uri"]
        data = [json.loads(line) for line in path.read_text(encoding="utf-8").splitlines() if line.strip()]
        if not data:
            raise ValueError(f"task {label}: no items in {path}")
        tasks.append({"label": label, "data": data, "random_baseline": baselines[label] / 100.0,
                      "meta": {"task_type": kind, "num_fewshot": int(entry["num_fewshot"][0]), "continuation_delimiter": entry.get("continuation_delimiter", " ")}})
    return tasks


def evaluate_bundle(logits_fn, encode, tasks: list[dict], *, max_per_task: int = -1, rank: int = 0, world: int = 1, group=None, shuffle_seed: int = 1337, **kw) -> dict:
    """Accuracy, centred accuracy ``(acc - b) / (1 - b)`` and their mean over the bundle.  Items are shuffled with a fixed
    seed BEFORE the ``max_per_task`` cut, so a subsample is the same on every run and every rank."""
    results, centered = {}, {}
    for task in tasks:
        data = list(task["data"])
        random.Random(shuffle_seed).shuffle(data)
        if max_per_task > 0:
            data = data[:max_per_task]
        counts = torch.tensor(evaluate_task(logits_fn, encode, data, task["meta"], rank=rank, world=world, **kw), dtype=torch.float64,
                              device=kw.get("device", "cpu"))
        if world > 1:
            torch.distributed.all_reduce(counts, group=group)
        results[task["label"]] = float(counts[0] / counts[1].clamp_min(1))
        centered[task["label"]] = (results[task["label"]] - task["random_baseline"]) / (1.0 - task["random_baseline"])
    return {"results": results, "centered_results": centered, "core_metric": sum(centered.values()) / max(len(centered), 1)}
