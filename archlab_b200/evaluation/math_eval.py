"""Sampled math benchmarks (integer-answer exams): stable per-sample seeds, final-answer scoring that records censoring,
unbiased pass@k, problem-level uncertainty, and a paired comparison of two models on the same exam.

* ``sample_seed`` depends on (seed, problem, sample index) only, so re-sharding a run over more workers draws the
  same samples.
* ``truncate_at_eos`` recovers the sample a corrected end-of-sequence set would have produced: nothing before the
  first EOS depends on where generation stopped, so no resampling (and no selection by correctness) is needed.
* ``score_sample`` grades the text after the reasoning block with the framework's answer verifier; a sample that hit
  the token budget may still score, but the fact is kept (``truncated``) so censoring shows in the report.
* ``summarize`` refuses unbalanced data: every expected problem needs exactly ``samples`` distinct draws.  pass@k uses
  the unbiased estimator; intervals resample PROBLEMS (repeats of a question are not independent exam questions); the
  first registered draw gets a Wilson interval.
* ``compare`` is the paired test on the first draw of every problem.
(Reference: src/archlab/evaluation/limite_math.py:84-194.)
"""
from __future__ import annotations

import hashlib
import math
import random
from collections import defaultdict
from statistics import NormalDist

from ..services.rewards import verify_math_answer
from .analysis import paired_statistics

GRADER = "archlab_b200.services.rewards.verify_math_answer"


def sample_seed(seed: int, problem_id: str, sample_index: int) -> int:
    if sample_index < 0:
        raise ValueError("sample index must be non-negative")
    digest = hashlib.sha256(f"{seed}:{problem_id}:{sample_index}".encode()).digest()
    return int.from_bytes(digest[:8], "big") % (2 ** 63 - 1)


def truncate_at_eos(token_ids: list[int], eos_token_ids) -> tuple[list[int], str]:
    eos = set(eos_token_ids)
    if not token_ids or not eos:
        raise ValueError("token and EOS lists must be non-empty")
    for i, t in enumerate(token_ids):
        if t in eos:
            return token_ids[:i + 1], "eos"
    return token_ids, "length"


def reasoning_closed(text: str) -> bool:
    """Every ``<think>`` has its ``</think>``; a surplus closing tag earlier cannot close a later block."""
    depth, i = 0, 0
    while True:
        a, b = text.find("<think>", i), text.find("</think>", i)
        if a < 0 and b < 0:
            return depth == 0
        if b < 0 or (0 <= a < b):
            depth, i = depth + 1, a + 7
        else:
            depth, i = max(0, depth - 1), b + 8


def score_sample(completion: str, answer: str, finish_reason: str, *, answer_range: tuple[int, int] = (0, 999)) -> dict:
    if finish_reason not in ("eos", "length"):
        raise ValueError("a benchmark sample ends naturally or at the token budget")
    if not answer.isdigit() or not answer_range[0] <= int(answer) <= answer_range[1]:
        raise ValueError("invalid reference answer for this exam")
    closed = reasoning_closed(completion)
    correct = closed and verify_math_answer(completion, answer).correct
    return {"correct": bool(correct), "reasoning_complete": closed, "natural_eos": finish_reason == "eos",
            "truncated": finish_reason == "length", "grader": GRADER}


def pass_at_k(correct: int, samples: int, k: int) -> float:
    if not 0 <= correct <= samples or not 1 <= k <= samples:
        raise ValueError("pass@k requires 0 <= correct <= samples and 1 <= k <= samples")
    wrong = samples - correct
    return 1.0 if wrong < k else 1.0 - math.comb(wrong, k) / math.comb(samples, k)


def wilson_interval(correct: int, total: int, confidence: float = 0.95) -> list[float]:
    if total < 1 or not 0 <= correct <= total:
        raise ValueError("a Wilson interval needs non-empty binary observations")
    z = NormalDist().inv_cdf(0.5 + confidence / 2)
    p, d = correct / total, 1 + z * z / total
    centre = (p + z * z / (2 * total)) / d
    half = z * math.sqrt(p * (1 - p) / total + z * z / (4 * total * total)) / d
    return [max(0.0, centre - half), min(1.0, centre + half)]


def _grouped(records, expected_ids, samples):
    if not expected_ids or len(set(expected_ids)) != len(expected_ids) or samples < 1:
        raise ValueError("a benchmark needs unique expected problems and a positive sample count")
    known = set(expected_ids)
    groups: dict[str, dict[int, dict]] = defaultdict(dict)
    for row in records:
        pid, idx = row["problem_id"], row["sample_index"]
        if pid not in known or type(idx) is not int or not 0 <= idx < samples:
            raise ValueError("record is outside the registered exam")
        if idx in groups[pid]:
            raise ValueError("duplicate benchmark response")
        if type(row["correct"]) is not bool:
            raise ValueError("correctness must be Boolean")
        groups[pid][idx] = row
    return groups


def summarize(records: list[dict], expected_ids: list[str], samples: int, *, ks=(1, 2, 4), bootstrap_draws: int = 10_000,
              seed: int = 0) -> dict:
    groups = _grouped(records, expected_ids, samples)
    done = [p for p in expected_ids if len(groups[p]) == samples]
    if len(done) != len(expected_ids):
        return {"complete": False, "completed_problems": len(done), "expected_problems": len(expected_ids),
                "recorded_samples": len(records), "expected_samples": len(expected_ids) * samples}
    rng = random.Random(seed)
    counts = [sum(r["correct"] for r in groups[p].values()) for p in expected_ids]
    n = len(expected_ids)
    out = {"complete": True, "problems": n, "samples_per_problem": samples, "responses": len(records), "correct_responses": sum(counts),
           "uncertainty_unit": "problem"}
    for k in (k for k in ks if k <= samples):
        per_problem = [pass_at_k(c, samples, k) for c in counts]
        means = sorted(sum(rng.choices(per_problem, k=n)) / n for _ in range(bootstrap_draws))
        out[f"pass_at_{k}"] = sum(per_problem) / n
        out[f"pass_at_{k}_interval"] = [means[int(0.025 * len(means))], means[min(len(means) - 1, int(0.975 * len(means)))]]
    first = [groups[p][0]["correct"] for p in expected_ids]
    lengths = sorted(r["generated_tokens"] for r in records)
    out.update(first_draw_correct=sum(first), first_draw_accuracy=sum(first) / n, first_draw_wilson=wilson_interval(sum(first), n),
               natural_eos_rate=sum(r["finish_reason"] == "eos" for r in records) / len(records),
               truncation_rate=sum(r["finish_reason"] == "length" for r in records) / len(records),
               mean_tokens=sum(lengths) / len(lengths), p50_tokens=lengths[len(lengths) // 2],
               p95_tokens=lengths[min(len(lengths) - 1, int(0.95 * len(lengths)))])
    return out


def compare(first: list[dict], second: list[dict], expected_ids: list[str]) -> dict:
    def first_draws(rows):
        picked = {r["problem_id"]: int(r["correct"]) for r in rows if r["sample_index"] == 0}
        if set(picked) != set(expected_ids):
            raise ValueError("a paired comparison needs the same complete benchmark on both sides")
        return [picked[p] for p in expected_ids]

    return paired_statistics(first_draws(first), first_draws(second))


# ---- a report over several models' sampled exams ------------------------------------------------------------------------
def completion_budget(prompt_tokens: int, requested: int, context: int) -> int:
    """The completion may spend the REMAINING native context: the prompt is never truncated to make room."""
    if not 0 < prompt_tokens < context or requested < 1:
        raise ValueError("the prompt does not fit the model's native context")
    return min(requested, context - prompt_tokens)


def read_complete_rows(path) -> list[dict]:
    """A live writer may have a half-written last line; a row counts only when its newline is there."""
    import json
    from pathlib import Path

    return [json.loads(line) for line in Path(path).read_text().split("\n")[:-1] if line.strip()]


def build_report(cases: list[dict], models: dict[str, dict], *, bootstrap_draws: int = 10_000) -> dict:
    """``cases``: ``{"id", "task"}``; ``models``: name -> ``{"records": [...], "samples_per_problem": n}`` where every record
    carries ``model``, ``problem_id``, ``sample_index``, ``correct``, ``finish_reason``, ``generated_tokens``.  Per model and
    exam (each task, and all tasks together): the first-draw summary and the repeated-draw summary; per pair of models
    whose first draws are complete: the paired test.  ``complete`` only when every repeated summary is."""
    from itertools import combinations

    exams = {task: [c["id"] for c in cases if c["task"] == task] for task in sorted({c["task"] for c in cases})}
    exams["all"] = [c["id"] for c in cases]
    report = {"format": "archlab-math-report-v1", "models": {}, "paired_first_draw": {}}
    complete = True
    for name, entry in models.items():
        rows = entry["records"]
        if any(r["model"] != name for r in rows):
            raise ValueError("a benchmark record belongs to another model than its registered output")
        per_exam = {}
        for task, ids in exams.items():
            subset = [r for r in rows if r["problem_id"] in set(ids)]
            per_exam[task] = {"first_draw": summarize([r for r in subset if r["sample_index"] == 0], ids, 1, bootstrap_draws=bootstrap_draws),
                              "repeated": summarize(subset, ids, entry["samples_per_problem"], bootstrap_draws=bootstrap_draws)}
            complete &= per_exam[task]["repeated"]["complete"]
        report["models"][name] = {"exams": per_exam, "recorded_samples": len(rows), "expected_samples": len(cases) * entry["samples_per_problem"]}
    for left, right in combinations(models, 2):
        pair = {}
        for task, ids in exams.items():
            if all(report["models"][m]["exams"][task]["first_draw"]["complete"] for m in (left, right)):
                pick = lambda m: [r for r in models[m]["records"] if r["problem_id"] in set(ids)]
                pair[task] = compare(pick(left), pick(right), ids)
        if pair:
            report["paired_first_draw"][f"{left} vs {right}"] = pair
    report["complete"] = bool(complete and models)
    return report


def markdown_report(report: dict) -> str:
    lines = ["# Sampled math evaluation", "", "Only completed exams are scored; partial response counts are progress, not accuracy.", "",
             "| Model | Exam | Draws / expected | First-draw accuracy | pass@1 | pass@4 | Truncated |", "| --- | --- | --- | --- | --- | --- | --- |"]
    for name, model in report["models"].items():
        for task, res in model["exams"].items():
            first, rep = res["first_draw"], res["repeated"]
            done = rep.get("responses", rep.get("recorded_samples", 0))
            expected = rep.get("expected_samples", rep.get("responses"))
            pct = lambda d, k: f"{d[k]:.1%}" if d.get("complete") and k in d else "pending"
            lines.append(f"| {name} | {task} | {done} / {expected} | {pct(first, 'first_draw_accuracy')} | {pct(rep, 'pass_at_1')} | {pct(rep, 'pass_at_4')} | {pct(rep, 'truncation_rate')} |")
    lines += ["", "The JSON report holds problem-cluster bootstrap intervals, Wilson intervals, paired tests, truncation rates and token lengths.", ""]
    return "\n".join(lines)
