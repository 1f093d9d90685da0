"""Matched-twin probe suites: sealing, prediction admission, twin-clustered summaries, calibration gate."""
import json

import pytest

from archlab_b200.evaluation import twin_suite as ts


def suite(tmp_path):
    rows = []
    for split, task in (("calibration", "retrieval"), ("test", "search")):
        for pair in range(6):
            for twin, expected in enumerate(("YES", "NO")):
                rid = f"{split}-{task}-{pair}-{twin}"
                rows.append({"id": rid, "pair_id": f"{split}-{task}-{pair}", "task": task, "level": 1, "split": split, "text": f"case {rid}", "input_ids": [1, 2, 3],
                             "token_audit": {"all_facts_in_long_window": pair < 4, "query_in_short_window": True}, "expected": expected})
    manifest = ts.seal_suite(tmp_path / "suite", rows, {"control_min_accuracy": 0.8})
    return rows, manifest


def run(tmp_path, name, rows, manifest, wrong=(), **marker):
    d = tmp_path / name
    d.mkdir()
    flip = {"YES": "NO", "NO": "YES"}
    preds = [{"id": r["id"], "text": flip[r["expected"]] if r["id"] in wrong else f" {r['expected']}\n"} for r in rows]
    (d / "predictions.jsonl").write_text("".join(json.dumps(p) + "\n" for p in preds))
    (d / "COMPLETE.json").write_text(json.dumps({"variant": name, "cases_sha256": manifest["cases_sha256"], "matched_training_tokens": 10 ** 9, "kind": "final", **marker}))
    return d


def test_summary_clusters_by_twin_and_gates_on_calibration(tmp_path):
    rows, manifest = suite(tmp_path)
    a = run(tmp_path, "normal", rows, manifest, wrong={"test-search-0-0", "test-search-1-1", "test-search-2-0"})
    b = run(tmp_path, "simplicial", rows, manifest, wrong={"test-search-0-0"})
    out = ts.summarize(tmp_path / "suite", {"normal": a, "simplicial": b}, draws=400)
    g = out["groups"]["test/search/1"]
    assert g["n"] == 12 and g["normal_accuracy"] == pytest.approx(9 / 12) and g["simplicial_accuracy"] == pytest.approx(11 / 12) and g["window_eligible"] == 8
    assert g["delta_pp"] == pytest.approx(100 * 2 / 12) and g["both_twins_paired_statistics"]["gained"] == 2 and g["invalid_outputs"] == [0, 0]
    assert g["twin_cluster_bootstrap_95pct_pp"][0] <= g["delta_pp"] <= g["twin_cluster_bootstrap_95pct_pp"][1]
    assert out["calibration_controls_pass"]
    c = run(tmp_path, "weak", rows, manifest, wrong={r["id"] for r in rows if r["split"] == "calibration" and r["id"].endswith("-0")})
    (tmp_path / "weak" / "COMPLETE.json").write_text(json.dumps({"variant": "weak", "cases_sha256": manifest["cases_sha256"], "matched_training_tokens": 10 ** 9, "kind": "final"}))
    assert not ts.summarize(tmp_path / "suite", {"normal": a, "weak": c}, draws=100)["calibration_controls_pass"]


def test_admission_of_predictions(tmp_path):
    rows, manifest = suite(tmp_path)
    a = run(tmp_path, "normal", rows, manifest)
    for name, kwargs, message in (("tiny", {"tiny": True}, "qualification-only"), ("other", {"cases_sha256": "x"}, "another suite"),
                                  ("late", {"matched_training_tokens": 5}, "not matched")):
        d = run(tmp_path, name, rows, manifest, **kwargs)
        with pytest.raises(ValueError, match=message):
            ts.summarize(tmp_path / "suite", {"normal": a, name: d}, draws=10)
    short = run(tmp_path, "short", rows[:-1], manifest)
    with pytest.raises(ValueError, match="missing, duplicate or extra"):
        ts.summarize(tmp_path / "suite", {"normal": a, "short": short}, draws=10)
    with pytest.raises(ValueError, match="wrong variant"):
        ts.summarize(tmp_path / "suite", {"normal": a, "renamed": a}, draws=10)
    (tmp_path / "suite" / "labels.json").write_text("[]")
    with pytest.raises(ValueError, match="sealed suite changed"):
        ts.summarize(tmp_path / "suite", {"normal": a, "short": short}, draws=10)
    audit = ts.token_audit("facts: a b c. query: is a b?", [(0, 6), (7, 8), (9, 10), (11, 13), (14, 20), (21, 23), (24, 25), (26, 28)],
                           {"facts": "a b c", "query": "is a b?"}, short_window=4, long_window=6)
    assert audit["prompt_tokens"] == 8 and audit["query_in_short_window"] and not audit["all_facts_in_long_window"]
