"""Sampled math benchmark rules: seeds, EOS correction, scoring with censoring, pass@k, balanced summaries, pairing."""
import math

import pytest

from archlab_b200.evaluation import math_eval as me


def test_seeds_are_stable_and_independent_of_sharding():
    assert me.sample_seed(7, "p1", 0) == me.sample_seed(7, "p1", 0) != me.sample_seed(7, "p1", 1)
    assert len({me.sample_seed(7, f"p{i}", j) for i in range(20) for j in range(4)}) == 80
    with pytest.raises(ValueError):
        me.sample_seed(7, "p", -1)


def test_eos_correction_and_reasoning_blocks():
    assert me.truncate_at_eos([5, 6, 2, 9, 2], [2, 3]) == ([5, 6, 2], "eos")
    assert me.truncate_at_eos([5, 6], [2]) == ([5, 6], "length")
    with pytest.raises(ValueError):
        me.truncate_at_eos([], [2])
    assert me.reasoning_closed("<think>a</think> 12") and not me.reasoning_closed("</think><think>a")
    assert me.reasoning_closed("no tags") and not me.reasoning_closed("<think><think></think>")


def test_scoring_records_censoring():
    ok = me.score_sample("<think>work</think>The answer is \\boxed{42}.", "42", "eos")
    assert ok["correct"] and ok["natural_eos"] and not ok["truncated"]
    late = me.score_sample("<think>work</think>\\boxed{42}", "42", "length")
    assert late["correct"] and late["truncated"]
    assert not me.score_sample("<think>still thinking \\boxed{42}", "42", "length")["correct"]      # thinking text is not mined
    assert not me.score_sample("\\boxed{41}", "42", "eos")["correct"]
    for bad in (("x", "42", "stop"), ("x", "1000", "eos"), ("x", "4.2", "eos")):
        with pytest.raises(ValueError):
            me.score_sample(*bad)


def test_pass_at_k_and_wilson():
    assert me.pass_at_k(0, 4, 2) == 0.0 and me.pass_at_k(4, 4, 1) == 1.0 and me.pass_at_k(3, 4, 2) == 1.0
    assert me.pass_at_k(1, 4, 2) == pytest.approx(1 - math.comb(3, 2) / math.comb(4, 2))
    with pytest.raises(ValueError):
        me.pass_at_k(1, 2, 3)
    lo, hi = me.wilson_interval(5, 10)
    assert 0.2 < lo < 0.5 < hi < 0.8 and me.wilson_interval(0, 10)[0] < 1e-12


def _records(pattern, samples=4):
    rows = []
    for pid, flags in pattern.items():
        for j in range(samples):
            rows.append({"problem_id": pid, "sample_index": j, "correct": bool(flags[j]), "finish_reason": "eos" if j else "length", "generated_tokens": 100 + j})
    return rows


def test_summaries_need_balanced_complete_exams():
    pattern = {"a": [1, 0, 0, 0], "b": [0, 0, 0, 0], "c": [1, 1, 1, 1]}
    rows = _records(pattern)
    s = me.summarize(rows, ["a", "b", "c"], 4, bootstrap_draws=200)
    assert s["complete"] and s["correct_responses"] == 5 and s["first_draw_correct"] == 2
    assert s["pass_at_1"] == pytest.approx((0.25 + 0 + 1) / 3) and s["pass_at_4"] == pytest.approx(2 / 3)
    assert s["pass_at_2_interval"][0] <= s["pass_at_2"] <= s["pass_at_2_interval"][1]
    assert s["truncation_rate"] == 0.25 and s["p50_tokens"] == 102
    partial = me.summarize(rows[:-1], ["a", "b", "c"], 4)
    assert partial == {"complete": False, "completed_problems": 2, "expected_problems": 3, "recorded_samples": 11, "expected_samples": 12}
    with pytest.raises(ValueError, match="duplicate"):
        me.summarize(rows + rows[:1], ["a", "b", "c"], 4)
    with pytest.raises(ValueError, match="outside"):
        me.summarize(rows, ["a", "b"], 4)
    with pytest.raises(ValueError, match="Boolean"):
        me.summarize([{**rows[0], "correct": 1}], ["a"], 4)


def test_paired_comparison_uses_the_first_draw():
    one = _records({"a": [1, 0, 0, 0], "b": [0, 1, 1, 1], "c": [0, 0, 0, 0]})
    two = _records({"a": [1, 0, 0, 0], "b": [1, 0, 0, 0], "c": [1, 0, 0, 0]})
    out = me.compare(one, two, ["a", "b", "c"])
    assert out["gained"] == 2 and out["lost"] == 0 and out["difference"] == pytest.approx(2 / 3)
    with pytest.raises(ValueError, match="same complete"):
        me.compare(one, two[4:], ["a", "b", "c"])


def test_multi_model_report_and_budget(tmp_path):
    cases = [{"id": "a", "task": "exam24"}, {"id": "b", "task": "exam24"}, {"id": "c", "task": "exam25"}]

    def records(model, pattern, drop=0):
        rows = [{"model": model, **r} for r in _records(pattern)]
        return rows[:len(rows) - drop]
    models = {"base": {"records": records("base", {"a": [0, 0, 0, 0], "b": [0, 1, 0, 0], "c": [0, 0, 0, 0]}), "samples_per_problem": 4},
              "tuned": {"records": records("tuned", {"a": [1, 1, 0, 1], "b": [1, 1, 1, 1], "c": [0, 0, 1, 0]}), "samples_per_problem": 4}}
    report = me.build_report(cases, models, bootstrap_draws=100)
    assert report["complete"] and set(report["models"]["base"]["exams"]) == {"exam24", "exam25", "all"}
    assert report["models"]["tuned"]["exams"]["exam24"]["repeated"]["pass_at_1"] == pytest.approx((0.75 + 1.0) / 2)
    assert report["paired_first_draw"]["base vs tuned"]["all"]["gained"] == 2
    text = me.markdown_report(report)
    assert "| tuned | exam24 | 8 / 8 | 100.0% | 87.5% | 100.0% | 25.0% |" in text
    models["tuned"]["records"] = records("tuned", {"a": [1, 1, 0, 1], "b": [1, 1, 1, 1], "c": [0, 0, 1, 0]}, drop=1)
    partial = me.build_report(cases, models, bootstrap_draws=50)
    assert not partial["complete"] and "pending" in me.markdown_report(partial)
    models["tuned"]["records"][0]["model"] = "other"
    with pytest.raises(ValueError, match="another model"):
        me.build_report(cases, models)
    assert me.completion_budget(1000, 131072, 131072) == 130072 and me.completion_budget(10, 50, 1000) == 50
    with pytest.raises(ValueError):
        me.completion_budget(2000, 10, 1000)
    live = tmp_path / "records.jsonl"
    live.write_text('{"a": 1}\n{"a": 2}\n{"a": 3')
    assert me.read_complete_rows(live) == [{"a": 1}, {"a": 2}]
