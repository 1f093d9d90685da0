"""Paired throughput comparison over matched updates; persistent curve crossover."""
import json
import math

import pytest

from archlab_b200.services import throughput_comparison as tc


def run(path, seconds, n=12, **edit):
    path.mkdir(parents=True)
    rows = [{"step": i, "loss": 3.0 - 0.01 * i, "seconds": seconds + 0.01 * (i % 3), "gradient_norm_before_clip": 1.0 + i, "supervised_tokens": 1000,
             "input_tokens": 1200, "consumed_supervised_tokens": 1000 * i, "learning_rate": 1e-3, "max_memory_allocated_gib": 40 + i} for i in range(1, n + 1)]
    for step, change in edit.items():
        rows[int(step[1:]) - 1].update(change)
    (path / "train.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
    (path / "validation.jsonl").write_text(json.dumps({"step": 0, "loss": 3.2}) + "\n" + json.dumps({"step": 10, "loss": 2.9}) + "\n")
    return path


def test_matched_window_ratio_and_interval(tmp_path):
    a, b = run(tmp_path / "a", 2.0), run(tmp_path / "b", 1.0)
    out = tc.compare_throughput(a, b, first=3, last=10, draws=500)
    assert out["paired_update_count"] == 8 and 1.9 < out["throughput_ratio"] < 2.0
    lo, hi = out["paired_bootstrap_ratio_interval_95"]
    assert lo <= out["throughput_ratio"] <= hi and out["baseline"]["peak_allocated_gib"] == 50
    assert out["other"]["supervised_targets_per_second"] == pytest.approx(8000 / out["other"]["total_update_seconds"])
    assert out["update_time_reduction_percent"] == pytest.approx((1 - 1 / out["throughput_ratio"]) * 100)


def test_unmatched_or_broken_runs_are_refused(tmp_path):
    a = run(tmp_path / "a", 2.0)
    with pytest.raises(ValueError, match="differs in learning_rate"):
        tc.compare_throughput(a, run(tmp_path / "b", 1.0, s5={"learning_rate": 2e-3}), first=3, last=10)
    with pytest.raises(ValueError, match="wait for the pre-declared step"):
        tc.compare_throughput(a, run(tmp_path / "c", 1.0, n=8), first=3, last=10)
    with pytest.raises(ValueError, match="non-finite"):
        tc.compare_throughput(a, run(tmp_path / "d", 1.0, s4={"loss": float("nan")}), first=3, last=10)
    e = run(tmp_path / "e", 1.0)
    (e / "validation.jsonl").write_text(json.dumps({"step": 0, "loss": 3.3}) + "\n")
    with pytest.raises(ValueError, match="initial held-out validation"):
        tc.compare_throughput(a, e, first=3, last=10)
    f = run(tmp_path / "f", 1.0)
    (f / "train.jsonl").write_text("".join((f / "train.jsonl").read_text().splitlines(keepends=True)[1:]))
    with pytest.raises(ValueError, match="uninterrupted"):
        tc.compare_throughput(a, f, first=3, last=10)
    with pytest.raises(ValueError, match="must follow"):
        tc.compare_throughput(a, a, first=1, last=10)


def test_crossover_needs_persistence():
    steps = list(range(10))
    a = [5.0] * 10
    b = [6, 4.9, 6, 6, 4.9, 4.8, 4.7, 6, 4.0, 4.0]
    assert tc.persistent_crossover(steps, a, b, persistence=3) == 4 and tc.persistent_crossover(steps, a, b, persistence=1) == 1
    assert tc.persistent_crossover(steps, a, b, persistence=4) is None
    assert tc.trailing_mean([1, 2, 3, 4], 2) == [1, 1.5, 2.5, 3.5]
    assert tc.median_step_seconds([(1, 10.0), (2, 12.0), (3, 15.0), (9, 99.0)], start_step=1, stop_step=3) == 2.5
    assert math.isnan(tc.median_step_seconds([(1, 10.0)], start_step=1, stop_step=3))
