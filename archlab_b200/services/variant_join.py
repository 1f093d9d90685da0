"""Joining two variants that were evaluated INDEPENDENTLY (each on its own node) into one comparison -- only after
both finished, and only if they were evaluated on the same thing.

Each variant directory holds ``COMPLETE.json`` (cursor, held-out language-model metrics, per-task choice accuracies),
``RUN_CONTRACT.json`` (what was evaluated: cursor, validation target count, digests of benchmark cases / jobs / prompts
and of the evaluator) and ``multiple-choice.jsonl`` (one scored case per line).  ``join`` refuses to produce anything
while an evaluation is unfinished or left a failure record, when the checkpoint cursors differ, when any contract digest
differs, or when the two case sets or their labels differ.  Then it pairs the cases, computes the paired choice summary
(``evaluation.paired_variants.choice_summary``), the cross-entropy difference on the held-out set, and writes
``COMPARISON.json``, a short ``REPORT.md`` table and its own ``COMPLETE.json``.  ``wait`` polls for up to a deadline.
(Reference: src/archlab/reporting/v41_scratch_eval_report.py:12-125.)
"""
from __future__ import annotations

import json
import time
from pathlib import Path

from ..contracts.substrate import atomic_write_json
from ..evaluation.paired_variants import choice_summary

CONTRACT_KEYS = ("cursor", "validation_targets", "benchmark_cases_sha256", "benchmark_jobs_digest", "prompts_sha256", "evaluator_sha256")
LM_KEYS = ("cross_entropy", "perplexity", "top1_token_accuracy", "top5_token_accuracy", "mean_predictive_entropy")


def ready(root, variants: tuple[str, str]) -> bool:
    root = Path(root)
    failures = [str(p) for v in variants for p in (root / v).glob("*failure.json")]
    if failures:
        raise RuntimeError(f"evaluation failed: {failures}")
    return all((root / v / "COMPLETE.json").exists() for v in variants)


def wait(root, variants: tuple[str, str], *, timeout_seconds: float = 4 * 3600, poll_seconds: float = 30.0, sleep=time.sleep) -> None:
    deadline = time.monotonic() + timeout_seconds
    while not ready(root, variants):
        if time.monotonic() > deadline:
            raise TimeoutError("the evaluations did not complete in time")
        sleep(poll_seconds)


def join(root, variants: tuple[str, str] = ("normal", "simplicial")) -> dict:
    root = Path(root)
    if not ready(root, variants):
        raise RuntimeError("both evaluations must complete first")
    a, b = variants
    done = {v: json.loads((root / v / "COMPLETE.json").read_text()) for v in variants}
    contracts = {v: json.loads((root / v / "RUN_CONTRACT.json").read_text()) for v in variants}
    if done[a]["cursor"] != done[b]["cursor"]:
        raise ValueError("checkpoint cursors differ")
    for key in CONTRACT_KEYS:
        if contracts[a][key] != contracts[b][key]:
            raise ValueError(f"evaluation contracts differ: {key}")
    rows = {v: {r["id"]: r for r in map(json.loads, filter(None, (root / v / "multiple-choice.jsonl").read_text().splitlines()))} for v in variants}
    if rows[a].keys() != rows[b].keys():
        raise ValueError("evaluated case ids differ")
    paired = []
    for key, ra in rows[a].items():
        rb = rows[b][key]
        if (ra["task"], ra["answer"]) != (rb["task"], rb["answer"]):
            raise ValueError("case labels differ")
        paired.append({"id": key, "task": ra["task"], "result": {a: ra["result"], b: rb["result"]}})
    choice = choice_summary(paired, (a, b))
    lm = {v: done[v]["heldout"] for v in variants}
    result = {"generated": time.time(), "passed": True, "cursor": done[a]["cursor"], "heldout": lm, "multiple_choice": choice,
              f"{a}_minus_{b}_ce": lm[a]["cross_entropy"] - lm[b]["cross_entropy"], "benchmark_overlap_with_training": "not assessed"}
    atomic_write_json(root / "COMPARISON.json", result)
    cursor = result["cursor"]
    lines = [f"Both variants evaluated at **{cursor.get('supervised_tokens', 0):,} supervised training tokens**, step {cursor.get('step')}, on matching inputs.", "",
             f"| Metric | {a} | {b} |", "|---|---:|---:|"]
    lines += [f"| held-out {k} | {lm[a][k]:.6f} | {lm[b][k]:.6f} |" for k in LM_KEYS if k in lm[a] and k in lm[b]]
    for task in choice:
        ta, tb = done[a]["multiple_choice"][task], done[b]["multiple_choice"][task]
        lines.append(f"| {task} accuracy ({ta['questions']} questions) | {100 * ta['accuracy']:.2f}% | {100 * tb['accuracy']:.2f}% |")
    lines += ["", "Small benchmark subsets do not establish a broad ranking; paired uncertainty statistics are in COMPARISON.json.", ""]
    (root / "REPORT.md").write_text("\n".join(lines))
    atomic_write_json(root / "COMPLETE.json", {"passed": True, "cursor": cursor, "comparison": "COMPARISON.json"})
    return result
