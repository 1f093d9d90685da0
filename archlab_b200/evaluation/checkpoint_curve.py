"""A two-way (or n-way) choice benchmark scored over the checkpoints of one run: one result file per checkpoint, reused
only when it was made with exactly this benchmark, tokenizer, template and model geometry; then a curve over tokens.

* ``encode_requests``: every (example, choice) becomes the tokens of ``context + delimiter + choice``; the choice's span
  is what the whole string adds to the context's own tokens (so tokenizer merges across the boundary are honoured);
  inputs are shifted by one for next-token scoring.
* ``score_requests``: batches in DATASET order (recurrent kernels may round differently under another batch shape, and a
  few nearly tied items would flip), right-padded, summed continuation log-likelihood per request; a non-finite score
  is an error.
* ``choice_result``: raw accuracy and accuracy with scores divided by the choice's character length, with binomial
  standard errors, plus the first few items verbatim for eyeballing.
* ``identity`` / ``load_cached``: a cached result counts only if its identity digest equals the current one and its
  own numbers are consistent; anything else is an error, never a silent reuse.
* ``aggregate``: the per-checkpoint results of one identity, ordered by training tokens.
(Reference: src/archlab/evaluation/qwen38_piqa.py:62-146,157-300,337-418.)
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

import torch

from ..contracts.substrate import atomic_write_json, sha256_file

SCHEMA = 1


@dataclass(frozen=True)
class Request:
    example: int
    choice: int
    input_ids: tuple[int, ...]
    continuation_ids: tuple[int, ...]
    continuation_text: str


def encode_requests(examples: list[dict], encode: Callable[[str], list[int]], *, template: str = "Question: {goal}\nAnswer:",
                    delimiter: str = " ") -> list[Request]:
    """``examples``: ``{"goal": str, "choices": [str, ...], "label": int}``."""
    out = []
    for i, ex in enumerate(examples):
        context = template.format(goal=ex["goal"])
        head = list(encode(context))
        for j, choice in enumerate(ex["choices"]):
            whole = list(encode(context + delimiter + choice))
            tail = whole[len(head):]
            if not head or not tail or whole[:len(head)] != head and len(whole) <= len(head):
                raise ValueError(f"empty token span at example {i}, choice {j}")
            out.append(Request(i, j, tuple((head + tail)[:-1]), tuple(tail), choice))
    return out


@torch.inference_mode()
def score_requests(logits_fn: Callable[[torch.Tensor], torch.Tensor], requests: list[Request], *, batch_size: int, pad_id: int,
                   device="cpu") -> list[float]:
    scores = [math.nan] * len(requests)
    for start in range(0, len(requests), batch_size):
        chunk = requests[start:start + batch_size]
        width = max(len(r.input_ids) for r in chunk)
        ids = torch.full((len(chunk), width), pad_id, dtype=torch.long, device=device)
        labels = torch.full_like(ids, -1)
        for row, r in enumerate(chunk):
            n, m = len(r.input_ids), len(r.continuation_ids)
            ids[row, :n] = torch.tensor(r.input_ids, device=device)
            labels[row, n - m:n] = torch.tensor(r.continuation_ids, device=device)
        logp = torch.log_softmax(logits_fn(ids).float(), -1)
        picked = logp.gather(-1, labels.clamp_min(0).unsqueeze(-1)).squeeze(-1) * labels.ge(0)
        for row, total in enumerate(picked.sum(-1).tolist()):
            scores[start + row] = total
    if not all(math.isfinite(s) for s in scores):
        raise RuntimeError("scoring produced a non-finite log-likelihood")
    return scores


def choice_result(examples: list[dict], requests: list[Request], scores: list[float], *, shown: int = 20) -> dict:
    table = [[math.nan] * len(ex["choices"]) for ex in examples]
    for r, s in zip(requests, scores, strict=True):
        table[r.example][r.choice] = s
    raw = norm = 0
    samples = []
    for i, (ex, row) in enumerate(zip(examples, table)):
        if any(math.isnan(v) for v in row):
            raise ValueError(f"example {i} lacks a score")
        best = max(range(len(row)), key=row.__getitem__)
        best_norm = max(range(len(row)), key=lambda j: row[j] / max(1, len(ex["choices"][j])))
        raw += best == ex["label"]
        norm += best_norm == ex["label"]
        if i < shown:
            samples.append({"goal": ex["goal"], "choices": ex["choices"], "label": ex["label"], "scores": row, "prediction": best})
    n = len(examples)
    se = lambda a: math.sqrt(a * (1 - a) / n)
    return {"examples": n, "accuracy": raw / n, "accuracy_stderr": se(raw / n), "accuracy_normalised": norm / n,
            "accuracy_normalised_stderr": se(norm / n), "samples": samples}


def _digest(value) -> str:
    return hashlib.sha256(json.dumps(value, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def identity(*, benchmark_file, tokenizer_sha256: str, template: str, delimiter: str, model_geometry: dict, batch_size: int,
             extra: dict | None = None) -> dict:
    body = {"schema": SCHEMA, "benchmark_sha256": sha256_file(benchmark_file), "tokenizer_sha256": tokenizer_sha256, "template": template,
            "delimiter": delimiter, "model_geometry": model_geometry, "batch_size": batch_size, **(extra or {})}
    return {**body, "sha256": _digest(body)}


def result_path(output_dir, iteration: int) -> Path:
    return Path(output_dir) / f"iter_{iteration:07d}.json"


def save_result(output_dir, iteration: int, tokens_per_iteration: int, result: dict, ident: dict, *, checkpoint: str, seconds: float) -> dict:
    body = {"iteration": iteration, "tokens": iteration * tokens_per_iteration, "checkpoint": checkpoint, "seconds": seconds,
            "identity": ident, **result}
    path = result_path(output_dir, iteration)
    path.parent.mkdir(parents=True, exist_ok=True)
    atomic_write_json(path, body)
    return body


def load_cached(output_dir, iteration: int, ident: dict, tokens_per_iteration: int) -> dict | None:
    """None if there is no result yet; the result if it belongs to this identity and is consistent; an error otherwise."""
    path = result_path(output_dir, iteration)
    if not path.exists():
        return None
    body = json.loads(path.read_text())
    if body.get("identity", {}).get("sha256") != ident["sha256"]:
        raise ValueError(f"{path.name} was made under another evaluation identity; move it away or use a new output directory")
    n = body.get("examples", 0)
    ok = (body.get("iteration") == iteration and body.get("tokens") == iteration * tokens_per_iteration and n > 0
          and all(0.0 <= body.get(k, -1) <= 1.0 for k in ("accuracy", "accuracy_normalised"))
          and abs(body["accuracy_stderr"] - math.sqrt(body["accuracy"] * (1 - body["accuracy"]) / n)) < 1e-9)
    if not ok:
        raise ValueError(f"{path.name} is inconsistent")
    return body


def aggregate(output_dir, iterations: list[int], ident: dict, tokens_per_iteration: int) -> list[dict]:
    rows = []
    for it in sorted(set(iterations)):
        body = load_cached(output_dir, it, ident, tokens_per_iteration)
        if body is None:
            raise FileNotFoundError(f"no result for iteration {it}")
        rows.append({k: body[k] for k in ("iteration", "tokens", "examples", "accuracy", "accuracy_stderr", "accuracy_normalised",
                                          "accuracy_normalised_stderr")})
    best = max(rows, key=lambda r: r["accuracy_normalised"]) if rows else None
    atomic_write_json(Path(output_dir) / "curve.json", {"identity_sha256": ident["sha256"], "rows": rows, "best": best})
    return rows


def run(output_dir, checkpoints: dict[int, str], load_model: Callable[[str], Callable], examples: list[dict], encode, ident: dict, *,
        tokens_per_iteration: int, batch_size: int, pad_id: int, device="cpu", template: str | None = None, delimiter: str | None = None) -> list[dict]:
    """Scores every checkpoint that has no valid cached result (``load_model(path)`` returns the logits function), then
    aggregates."""
    import time

    requests = encode_requests(examples, encode, template=template or ident["template"], delimiter=delimiter if delimiter is not None else ident["delimiter"])
    for it, path in sorted(checkpoints.items()):
        if load_cached(output_dir, it, ident, tokens_per_iteration) is not None:
            continue
        t0 = time.monotonic()
        scores = score_requests(load_model(path), requests, batch_size=batch_size, pad_id=pad_id, device=device)
        save_result(output_dir, it, tokens_per_iteration, choice_result(examples, requests, scores), ident, checkpoint=str(path),
                    seconds=time.monotonic() - t0)
    return aggregate(output_dir, list(checkpoints), ident, tokens_per_iteration)
