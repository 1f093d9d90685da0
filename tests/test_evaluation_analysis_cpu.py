import json
import random

import numpy as np
import pytest

from archlab_b200.evaluation import analysis as A


def test_ladder_candidates_and_ledger(tmp_path):
    ex = tmp_path / "exports"
    for s, ok in ((100, True), (200, True), (250, False), (300, True)):
        d = ex / f"run-step{s}"
        d.mkdir(parents=True)
        if ok:
            (d / "EXPORTED").write_text("")
    assert A.exported_steps(ex, "run") == [100, 200, 300]
    fixed = tmp_path / "base"
    fixed.mkdir()
    plan = {"points": [{"label": "base", "model": str(fixed), "curve": "c", "step": 0},
                       {"every": {"exports": str(ex), "prefix": "run", "every": 100, "curve": "c"}},
                       {"newest": {"exports": str(ex), "prefix": "run", "every": 150, "curve": "c"}}]}
    labels = [p["label"] for p in A.ladder_candidates(plan, set())]
    assert labels == ["base", "run-step100", "run-step200", "run-step300"]
    assert [p["label"] for p in A.ladder_candidates(plan, {"base", "run-step100", "run-step200"})] == ["run-step300"]
    led = A.PointLedger(tmp_path / "ledger.jsonl")
    assert led.record("base", score=0.5) and not led.record("base", score=0.9) and led.done() == {"base"}


def test_paired_statistics_and_selection():
    base = [0, 0, 1, 1, 0, 1, 0, 0]
    adapted = [1, 1, 1, 1, 0, 0, 1, 1]
    s = A.paired_statistics(base, adapted)
    assert s["gained"] == 4 and s["lost"] == 1 and s["difference"] == pytest.approx(3 / 8)
    assert s["sign_test_p"] == pytest.approx(2 * (1 + 5) / 32) and s["interval"][0] < s["difference"] < s["interval"][1]
    with pytest.raises(ValueError):
        A.paired_statistics([0, 1], [1])
    rows = [{"suite": "a", "id": i} for i in range(10)] + [{"suite": "b", "id": i} for i in range(3)]
    pick = A.select_cases(rows, limits={"a": 4, "b": 2}, seed=1)
    assert len(pick) == 6 and pick == A.select_cases(list(reversed(rows)), limits={"a": 4, "b": 2}, seed=1)
    with pytest.raises(ValueError):
        A.select_cases(rows, limits={"b": 5}, seed=1)


def test_pair_search_twins_have_exact_answers():
    rng = random.Random(0)
    for _ in range(20):
        t = A.make_twins(rng, earlier_count=12, recent_count=3)
        assert A.witnesses(t["recent"], t["no"], t["target"], 97) == []
        assert A.witnesses(t["recent"], t["yes"], t["target"], 97) == [t["witness"]]
        assert sum(a != b for a, b in zip(t["no"], t["yes"])) == 1


def test_replay_window_scores_only_generated_tokens():
    prompt, resp = np.arange(10), np.arange(100, 112)
    gen = np.array([1, 1, 0, 0, 1, 1, 1, 0, 1, 1, 1, 1])
    tokens, mask, n = A.replay_window(prompt, resp, gen, 12)
    assert tokens.tolist() == list(range(4, 10)) + list(range(100, 106)) and len(mask) == 11
    assert mask[:5].sum() == 0 and mask[5:].tolist() == [True, True, False, False, True, True] and n == 4


def test_rollout_accounting(tmp_path):
    def sess(step, k, task, reward):
        d = tmp_path / f"step_{step}" / f"session-{k}"
        d.mkdir(parents=True)
        (d / "session.json").write_text(json.dumps({"dataset_index": task, "reward_score": reward, "num_turns": 3}))
    k = 0
    for step, task, rewards in [(1, 0, [0, 0]), (1, 1, [0, 1]), (2, 0, [1, 1]), (2, 2, [0, 0]), (3, 1, [1, 1])]:
        for r in rewards:
            sess(step, k, task, r)
            k += 1
    rows = A.read_sessions(tmp_path)
    w = A.waste(rows)
    assert w["groups"] == 5 and w["all_failed"] == 2 and w["all_solved"] == 2 and w["informative"] == 1
    lg = A.learning(rows)
    assert lg["tasks"] == 2 and lg["gain"] == pytest.approx((1.0 + 0.5) / 2)
    keep = A.learnable_rows(rows, 5, "snap", recheck=0.0)
    assert keep == [0, 1, 3, 4]                                   # task 2 failed on its last visit, 3 and 4 never seen
