"""Fixed-grid agentic evaluation: missing cells stay missing, contracts are bound, differences are task-paired."""
import json

import pytest

from archlab_b200.evaluation import agentic_grid as ag

TASKS, SEEDS = ["t0", "t1", "t2"], [101, 211]


def rows(pattern, missing=()):
    out = []
    for t, rewards in pattern.items():
        for s, r in zip(SEEDS, rewards):
            if (t, s) in missing:
                out.append({"task": t, "seed": s, "status": "missing", "reward": None})
            else:
                out.append({"task": t, "seed": s, "status": "scored", "reward": float(r), "termination": "completed", "generated_tokens": 100, "seconds": 2.0})
    return out


def test_summaries_exist_only_for_complete_grids():
    full = ag.summarize(rows({"t0": [1, 1], "t1": [0, 1], "t2": [0, 0]}), TASKS, SEEDS, bootstrap=300)
    assert full["complete"] and full["pass_at_1"] == pytest.approx(0.5) and full["success_at_k"] == pytest.approx(2 / 3) and full["preliminary"]
    assert full["task_bootstrap_95ci"][0] <= 0.5 <= full["task_bootstrap_95ci"][1] and full["generated_tokens"] == 600
    partial = ag.summarize(rows({"t0": [1, 1], "t1": [0, 1], "t2": [0, 0]}, missing={("t2", 211)}), TASKS, SEEDS)
    assert not partial["complete"] and partial["pass_at_1"] is None and partial["missing_samples"] == 1 and partial["infrastructure_attempts"] == 1
    assert partial["provisional_complete_task_pass_at_1"] == pytest.approx(0.75) and partial["per_task"]["t2"] == {"scored": 1, "successes": 0.0, "expected": 2}
    with pytest.raises(ValueError, match="outside the declared grid"):
        ag.summarize(rows({"t9": [1, 1]}), TASKS, SEEDS)
    with pytest.raises(ValueError, match="duplicate"):
        ag.summarize(rows({"t0": [1, 1]}) * 2, TASKS, SEEDS)
    with pytest.raises(ValueError, match="binary"):
        ag.summarize([{"task": "t0", "seed": 101, "status": "scored", "reward": 0.5}], TASKS, SEEDS)
    assert ag.sample_seed("t0", 101) == ag.sample_seed("t0", 101) != ag.sample_seed("t0", 211)


def test_invocations_can_only_grow_their_seed_list(tmp_path):
    path = tmp_path / "invocation.json"
    base = {"model": "ckpt-10", "tasks_sha256": "x", "seeds": [101, 211], "scope": "pilot"}
    ag.bind_invocation(path, base)
    ag.bind_invocation(path, {**base, "seeds": [101, 211, 307], "scope": "full"})
    assert json.loads(path.read_text())["seeds"] == [101, 211, 307] and len(list(tmp_path.glob("invocation-*.json"))) == 1
    for bad in ({**base, "model": "ckpt-20"}, {**base, "seeds": [211, 101, 307]}, {**base, "seeds": [101]}):
        with pytest.raises(ValueError, match="different evaluation contract"):
            ag.bind_invocation(path, bad)


def test_paired_difference_and_outcome_labels():
    a, b = rows({"t0": [0, 0], "t1": [0, 1], "t2": [0, 0]}), rows({"t0": [1, 1], "t1": [0, 1], "t2": [1, 0]})
    d = ag.paired_difference(a, b, TASKS, SEEDS, bootstrap=300)
    assert d["delta_pass_at_1"] == pytest.approx(0.5) and d["task_paired_95ci"][0] >= 0
    with pytest.raises(ValueError, match="both grids"):
        ag.paired_difference(a[:-1], b, TASKS, SEEDS)
    assert ag.error_outcome(TimeoutError("session exceeded wall timeout"))["termination"] == "wall_budget_unclassified"
    assert ag.error_outcome(ConnectionError("reset"))["termination"] == "infrastructure_or_unclassified"
    assert ag.policy_cap_reason({"agent_completed": True}, 12) == "none" and ag.policy_cap_reason({}, 300) == "turn_limit"
    assert ag.policy_cap_reason({"result": "Maximum context length exceeded", "agent_status": "ModelQueryError"}, 5) == "context_limit"
    assert ag.policy_cap_reason({"result": "stopped"}, 5) == "unfinished_other"
    with pytest.raises(RuntimeError, match="ungradable"):
        ag.policy_cap_reason({"agent_status": "ModelQueryError", "result": "502 bad gateway"}, 5)
