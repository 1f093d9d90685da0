"""Two model variants on the same held-out windows: token-level agreement and a clustered paired uncertainty.

``score_window(logits_a, logits_b, labels)`` reduces one window on the device: per variant summed NLL, top-1 / top-5 hits
and predictive entropy over the supervised positions, the two KL divergences between the variants' predictive
distributions, and how often their argmax agrees.  Only sums leave the device, so windows of any length aggregate
exactly.  ``aggregate`` turns a list of window records into cross-entropy, perplexity, accuracies, mean KLs and
agreement; ``summary`` adds break-downs (by reasoning mode, with / without tools) and a paired percentile bootstrap in
which the resampling unit is the PROBLEM (all windows of one problem move together), because windows of one problem are
not independent.  ``choice_summary`` is the paired analysis of multiple-choice results per task.
(Reference: src/archlab/evaluation/deepseek_v41_compare_metrics.py:14-129.)
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .analysis import paired_statistics


@torch.no_grad()
def score_window(logits_a: torch.Tensor, logits_b: torch.Tensor, labels: torch.Tensor, names: tuple[str, str] = ("a", "b")) -> dict:
    """logits [T, V] each, labels [T] with -1 = unsupervised."""
    keep = labels.ge(0)
    n = int(keep.sum())
    if n == 0:
        raise ValueError("a window without supervised targets")
    y = labels[keep]
    out = {"targets": n}
    logp = []
    for name, logits in zip(names, (logits_a, logits_b)):
        lp = torch.log_softmax(logits[keep].float(), -1)
        logp.append(lp)
        top5 = lp.topk(min(5, lp.shape[-1]), -1).indices
        out[name] = {"nll": float(-lp.gather(-1, y[:, None]).sum()), "top1": int((top5[:, 0] == y).sum()), "top5": int((top5 == y[:, None]).any(-1).sum()),
                     "entropy": float(-(lp.exp() * lp).sum())}
    a, b = logp
    out[f"{names[0]}_to_{names[1]}_kl_sum"] = float((a.exp() * (a - b)).sum())
    out[f"{names[1]}_to_{names[0]}_kl_sum"] = float((b.exp() * (b - a)).sum())
    out["argmax_agreement_count"] = int((a.argmax(-1) == b.argmax(-1)).sum())
    return out


def aggregate(records: list[dict], names: tuple[str, str] = ("a", "b")) -> dict:
    total = sum(r["targets"] for r in records)
    if not total:
        raise ValueError("empty evaluation")
    out = {"windows": len(records), "supervised_targets": total, "variants": {}}
    for v in names:
        nll = sum(r[v]["nll"] for r in records) / total
        out["variants"][v] = {"cross_entropy": nll, "perplexity": math.exp(nll), "top1_token_accuracy": sum(r[v]["top1"] for r in records) / total,
                              "top5_token_accuracy": sum(r[v]["top5"] for r in records) / total,
                              "mean_predictive_entropy": sum(r[v]["entropy"] for r in records) / total}
    for field in (f"{names[0]}_to_{names[1]}_kl", f"{names[1]}_to_{names[0]}_kl"):
        out[field] = sum(r[field + "_sum"] for r in records) / total
    out["token_argmax_agreement"] = sum(r["argmax_agreement_count"] for r in records) / total
    out[f"{names[1]}_minus_{names[0]}_ce"] = out["variants"][names[1]]["cross_entropy"] - out["variants"][names[0]]["cross_entropy"]
    return out


def summary(records: list[dict], names: tuple[str, str] = ("a", "b"), *, seed: int = 0, replicates: int = 10_000) -> dict:
    """Records additionally carry ``problem_sha256`` and optionally ``mode`` and ``has_tools``."""
    a, b = names
    out = {"overall": aggregate(records, names), "by_mode": {}, "by_tools": {}}
    for mode in sorted({r["mode"] for r in records if "mode" in r}):
        out["by_mode"][mode] = aggregate([r for r in records if r.get("mode") == mode], names)
    for tools in (False, True):
        part = [r for r in records if "has_tools" in r and bool(r["has_tools"]) == tools]
        if part:
            out["by_tools"]["tools" if tools else "no_tools"] = aggregate(part, names)
    clusters: dict[str, np.ndarray] = {}
    for r in records:
        acc = clusters.setdefault(r["problem_sha256"], np.zeros(4))
        acc += np.array([r["targets"], r[b]["nll"] - r[a]["nll"], r[b]["top1"] - r[a]["top1"], r[b]["top5"] - r[a]["top5"]], dtype=np.float64)
    values = np.stack(list(clusters.values()))
    rng = np.random.default_rng(seed)
    draws = values[rng.integers(0, len(values), (replicates, len(values)))].sum(1)
    bounds = np.quantile(draws[:, 1:] / draws[:, :1], [0.025, 0.975], axis=0)
    out["paired_uncertainty"] = {"method": "paired percentile bootstrap clustered by problem hash", "problem_clusters": len(clusters),
                                 "replicates": replicates, "seed": seed, "delta_definition": f"{b} minus {a}",
                                 "cross_entropy_delta_interval": bounds[:, 0].tolist(), "top1_accuracy_delta_interval_pp": (bounds[:, 1] * 100).tolist(),
                                 "top5_accuracy_delta_interval_pp": (bounds[:, 2] * 100).tolist()}
    return out


def score_choice_vector(case: dict, values: list[float]) -> dict:
    """``case``: ``{"id", "choices": [...], "answer": int, "length_normalised": bool}`` (knowledge quizzes with letter
    answers are not length-normalised)."""
    lengths = [len(c) for c in case["choices"]] if case.get("length_normalised", True) else [1] * len(case["choices"])
    if any(n <= 0 for n in lengths):
        raise ValueError("empty choice text")
    if len(values) != len(lengths) or any(v is None or not math.isfinite(v) for v in values):
        raise ValueError(f"incomplete or non-finite choice scores: {case['id']}")
    norm = [v / n for v, n in zip(values, lengths)]
    pred, pred_norm = max(range(len(values)), key=values.__getitem__), max(range(len(values)), key=norm.__getitem__)
    return {"prediction": pred, "normalized_prediction": pred_norm, "accuracy": int(pred == case["answer"]), "accuracy_norm": int(pred_norm == case["answer"])}


def choice_summary(records: list[dict], names: tuple[str, str] = ("a", "b")) -> dict:
    """Records: ``{"task", "id", "result": {variant: score_choice_vector(...)}}``."""
    a, b = names
    out = {}
    for task in sorted({r["task"] for r in records}):
        rows = [r for r in records if r["task"] == task]
        out[task] = {metric: {**paired_statistics([r["result"][a][metric] for r in rows], [r["result"][b][metric] for r in rows]),
                              "delta_definition": f"{b} minus {a}"} for metric in ("accuracy", "accuracy_norm")}
        out[task]["samples"] = len(rows)
        out[task]["prediction_agreement"] = sum(r["result"][a]["prediction"] == r["result"][b]["prediction"] for r in rows) / len(rows)
        out[task]["overlaps_with_consumed_training"] = [r["id"] for r in rows if r.get("exact_overlap_consumed_training")]
    return out
