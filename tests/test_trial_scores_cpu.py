"""Harness job scoring: errored trials count as zero, unfinished jobs are not scored."""
import json

import pytest

from archlab_b200.evaluation.trial_scores import complete_job, score_trials


def trial(job, name, reward=None, error=None):
    d = job / name
    d.mkdir(parents=True)
    (d / "result.json").write_text(json.dumps({"task_name": name, "verifier_result": None if reward is None else {"rewards": {"reward": reward}},
                                               "exception_info": None if error is None else {"exception_type": error}}))


def test_scores(tmp_path):
    job = tmp_path / "jobs" / "label" / "run-1"
    for i in range(6):
        trial(job, f"t{i}", reward=1.0 if i < 3 else 0.0)
    trial(job, "crashed", error="AgentTimeoutError")
    trial(job, "crashed2", error="AgentTimeoutError")
    s = score_trials(job, bootstrap=500, valid={"t0", "t1", "t5", "crashed"})
    assert s["trials"] == 8 and s["solved"] == 3 and s["mean_reward"] == pytest.approx(3 / 8) and s["errors"] == {"AgentTimeoutError": 2}
    assert s["ci95"][0] <= s["mean_reward"] <= s["ci95"][1] and s["solved_tasks"] == ["t0", "t1", "t2"]
    assert s["oracle_valid"] == {"tasks": 4, "mean_reward": 0.5}
    with pytest.raises(ValueError, match="no trials"):
        score_trials(tmp_path / "empty")


def test_only_finished_jobs_are_found(tmp_path):
    jobs = tmp_path / "jobs"
    for name, running in (("run-a", 2), ("run-b", 0)):
        (jobs / "label" / name).mkdir(parents=True)
        (jobs / "label" / name / "result.json").write_text(json.dumps({"stats": {"n_running_trials": running, "n_pending_trials": 0}}))
    assert complete_job(jobs, "label").name == "run-b" and complete_job(jobs, "other") is None
