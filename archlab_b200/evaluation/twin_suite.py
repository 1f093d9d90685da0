"""Matched-twin probe suites (YES / NO questions that come in pairs differing in one fact) evaluated on two variants.

``seal_suite`` freezes the public cases (text, token ids, a token audit saying how far facts and query sit from the
first predicted token) separately from the labels, with SHA-256 of both in ``MANIFEST.json``: predictions are produced
from ``cases.json`` alone.  ``summarize`` refuses a changed suite, predictions of the wrong variant / suite / a
qualification-only run, missing, duplicate or extra predictions, and variants that were not matched at the same training
phase and token count.  Per (split, task, level) it reports both accuracies, invalid outputs (anything but YES / NO), the
difference with a bootstrap that resamples WHOLE twins, the paired statistics of "both twins correct", and how many cases
were window-eligible (all facts inside the long window, the query inside the short window).  ``calibration_controls_pass``
is false when either variant falls under the configured accuracy on the retrieval / arithmetic calibration groups: a
failure there means a deficit elsewhere must not be attributed to the mechanism under study.
(Reference: src/archlab/evaluation/reasoning.py:142-281; twin generation: ``evaluation.analysis.make_twins``.)
"""
from __future__ import annotations

import json
import random
from collections import defaultdict
from pathlib import Path

from ..contracts.substrate import sha256_file
from .analysis import paired_statistics

FORMAT = "archlab-matched-twin-suite-v1"
META = ("id", "pair_id", "task", "level", "split")


def token_audit(prompt: str, offsets: list[tuple[int, int]], spans: dict[str, str], *, short_window: int, long_window: int) -> dict:
    """Distances (in tokens) of the named text spans from the first predicted token."""
    n = len(offsets)
    distances = {}
    for name, text in spans.items():
        start = prompt.index(text)
        stop = start + len(text)
        hit = [i for i, (a, b) in enumerate(offsets) if b > start and a < stop]
        if not hit:
            raise ValueError("token offsets do not cover the span")
        distances[name] = {"first": n - 1 - min(hit), "last": n - 1 - max(hit)}
    return {"prompt_tokens": n, "distances_from_first_prediction": distances,
            "all_facts_in_long_window": distances["facts"]["first"] < long_window, "query_in_short_window": distances["query"]["first"] < short_window}


def seal_suite(output, rows: list[dict], config: dict) -> dict:
    """``rows``: ``{id, pair_id, task, level, split, text, input_ids, token_audit, expected}``."""
    output = Path(output)
    output.mkdir(parents=True, exist_ok=False)
    if len({r["id"] for r in rows}) != len(rows) or any(r["expected"] not in ("YES", "NO") for r in rows):
        raise ValueError("case ids must be unique and answers YES or NO")
    public = [{**{k: r[k] for k in META}, "text": r["text"], "input_ids": r["input_ids"], "token_audit": r["token_audit"]} for r in rows]
    labels = [{**{k: r[k] for k in META}, "expected": r["expected"]} for r in rows]
    (output / "cases.json").write_text(json.dumps(public, indent=1) + "\n")
    (output / "labels.json").write_text(json.dumps(labels, indent=1) + "\n")
    manifest = {"format": FORMAT, "config": config, "cases_sha256": sha256_file(output / "cases.json"), "labels_sha256": sha256_file(output / "labels.json"),
                "rows": len(rows), "caveat": "frozen zero-shot probes; a window audit is not a proof of a one-layer computation"}
    (output / "MANIFEST.json").write_text(json.dumps(manifest, indent=1) + "\n")
    return manifest


def summarize(bundle, runs: dict[str, Path], *, draws: int = 10_000, seed: int = 20260929) -> dict:
    """``runs``: variant name -> directory with ``COMPLETE.json`` and ``predictions.jsonl`` (exactly two variants)."""
    bundle = Path(bundle)
    manifest = json.loads((bundle / "MANIFEST.json").read_text())
    for key in ("cases", "labels"):
        if sha256_file(bundle / f"{key}.json") != manifest[f"{key}_sha256"]:
            raise ValueError("the sealed suite changed")
    labels = json.loads((bundle / "labels.json").read_text())
    cases = {r["id"]: r for r in json.loads((bundle / "cases.json").read_text())}
    if len(runs) != 2:
        raise ValueError("a comparison has exactly two variants")
    names, predictions, markers = list(runs), [], []
    for variant, directory in runs.items():
        marker = json.loads((Path(directory) / "COMPLETE.json").read_text())
        if marker["variant"] != variant or marker.get("tiny"):
            raise ValueError("wrong variant or qualification-only predictions")
        if marker["cases_sha256"] != manifest["cases_sha256"]:
            raise ValueError("predictions belong to another suite")
        markers.append(marker)
        rows = [json.loads(line) for line in (Path(directory) / "predictions.jsonl").read_text().splitlines() if line.strip()]
        indexed = {r["id"]: r for r in rows}
        if len(indexed) != len(rows) or set(indexed) != set(cases):
            raise ValueError("missing, duplicate or extra predictions")
        predictions.append(indexed)
    if any(markers[0][k] != markers[1][k] for k in ("matched_training_tokens", "kind")):
        raise ValueError("the checkpoints are not matched at the same phase and token count")
    groups = defaultdict(list)
    for label in labels:
        groups[(label["split"], label["task"], label["level"])].append(label)
    result = {}
    for (split, task, level), rows in sorted(groups.items()):
        scores, invalid = [[], []], [0, 0]
        twins: dict = defaultdict(lambda: [[], []])
        for row in rows:
            for arm, pred in enumerate(predictions):
                answer = pred[row["id"]]["text"].strip()
                ok = int(answer == row["expected"])
                invalid[arm] += int(answer not in ("YES", "NO"))
                scores[arm].append(ok)
                twins[row["pair_id"]][arm].append(ok)
        both = [[int(all(t[arm])) for t in twins.values()] for arm in (0, 1)]
        rng = random.Random(seed)
        per_twin = [(sum(t[1]) - sum(t[0])) / max(1, len(t[0])) for t in twins.values()]
        deltas = sorted(100 * sum(rng.choices(per_twin, k=len(per_twin))) / len(per_twin) for _ in range(draws))
        result[f"{split}/{task}/{level}"] = {
            "n": len(rows), f"{names[0]}_accuracy": sum(scores[0]) / len(rows), f"{names[1]}_accuracy": sum(scores[1]) / len(rows), "invalid_outputs": invalid,
            "delta_pp": 100 * (sum(scores[1]) - sum(scores[0])) / len(rows), "twin_cluster_bootstrap_95pct_pp": [deltas[int(0.025 * draws)], deltas[int(0.975 * draws) - 1]],
            "both_twins_paired_statistics": paired_statistics(*both),
            "window_eligible": sum(cases[r["id"]]["token_audit"]["all_facts_in_long_window"] and cases[r["id"]]["token_audit"]["query_in_short_window"] for r in rows)}
    floor = manifest["config"].get("control_min_accuracy", 0.0)
    controls = [v for k, v in result.items() if k.startswith("calibration/") and any(t in k for t in ("retrieval", "arithmetic"))]
    return {"cases_sha256": manifest["cases_sha256"], "variants": names, "groups": result,
            "calibration_controls_pass": all(min(v[f"{names[0]}_accuracy"], v[f"{names[1]}_accuracy"]) >= floor for v in controls),
            "interpretation": "exploratory frozen zero-shot probes; no deficit is attributed to the mechanism if the calibration controls fail; "
                              "task comparisons are descriptive, without a multiple-comparison adjustment",
            "bootstrap_note": "whole twins are resampled; percentile intervals can degenerate at zero discordance"}
