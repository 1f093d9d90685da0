"""Joining two independently evaluated variants: matching contracts are a precondition."""
import json

import pytest

from archlab_b200.services import variant_join as vj

CONTRACT = {"cursor": {"step": 100, "supervised_tokens": 10 ** 9}, "validation_targets": 1000, "benchmark_cases_sha256": "c", "benchmark_jobs_digest": "j",
            "prompts_sha256": "p", "evaluator_sha256": "e"}


def variant(root, name, ce, correct, **edit):
    d = root / name
    d.mkdir(parents=True)
    cases = [{"id": f"q{i}", "task": "quiz", "answer": i % 2, "result": {"prediction": i % 2 if i < correct else 1 - i % 2, "accuracy": int(i < correct),
                                                                         "accuracy_norm": int(i < correct)}} for i in range(10)]
    (d / "multiple-choice.jsonl").write_text("".join(json.dumps(c) + "\n" for c in edit.get("cases", cases)))
    (d / "RUN_CONTRACT.json").write_text(json.dumps({**CONTRACT, **edit.get("contract", {})}))
    if edit.get("complete", True):
        (d / "COMPLETE.json").write_text(json.dumps({"cursor": edit.get("cursor", CONTRACT["cursor"]), "heldout": {"cross_entropy": ce, "perplexity": 2.718 ** ce},
                                                     "multiple_choice": {"quiz": {"questions": 10, "accuracy": correct / 10}}}))
    return cases


def test_join_writes_comparison_and_report(tmp_path):
    variant(tmp_path, "normal", 2.5, 5)
    variant(tmp_path, "simplicial", 2.4, 8)
    out = vj.join(tmp_path)
    assert out["normal_minus_simplicial_ce"] == pytest.approx(0.1) and out["multiple_choice"]["quiz"]["accuracy"]["gained"] == 3
    report = (tmp_path / "REPORT.md").read_text()
    assert "1,000,000,000 supervised training tokens" in report and "| quiz accuracy (10 questions) | 50.00% | 80.00% |" in report
    assert json.loads((tmp_path / "COMPLETE.json").read_text())["comparison"] == "COMPARISON.json"


def test_refusals(tmp_path):
    variant(tmp_path / "a", "normal", 2.5, 5)
    variant(tmp_path / "a", "simplicial", 2.4, 8, complete=False)
    with pytest.raises(RuntimeError, match="must complete first"):
        vj.join(tmp_path / "a")
    with pytest.raises(TimeoutError):
        vj.wait(tmp_path / "a", ("normal", "simplicial"), timeout_seconds=0.0, poll_seconds=0.0, sleep=lambda s: None)
    (tmp_path / "a" / "simplicial" / "oom-failure.json").write_text("{}")
    with pytest.raises(RuntimeError, match="evaluation failed"):
        vj.join(tmp_path / "a")
    variant(tmp_path / "b", "normal", 2.5, 5)
    variant(tmp_path / "b", "simplicial", 2.4, 8, contract={"prompts_sha256": "other"})
    with pytest.raises(ValueError, match="contracts differ: prompts_sha256"):
        vj.join(tmp_path / "b")
    variant(tmp_path / "c", "normal", 2.5, 5)
    variant(tmp_path / "c", "simplicial", 2.4, 8, cursor={"step": 90, "supervised_tokens": 9})
    with pytest.raises(ValueError, match="cursors differ"):
        vj.join(tmp_path / "c")
    cases = variant(tmp_path / "d", "normal", 2.5, 5)
    variant(tmp_path / "d", "simplicial", 2.4, 8, cases=cases[:-1])
    with pytest.raises(ValueError, match="case ids differ"):
        vj.join(tmp_path / "d")
