"""Code rewards: verdicts are admissible, infrastructure failures and inconsistent records are not; truncation is not success."""
import pytest

from archlab_b200.services.code_verdict import RewardInfrastructureError, classify_stop, require_code_verdict

TASK = {"dataset_type": "opensource-code", "instance_id": "task"}


@pytest.mark.parametrize("code,reward", [(0, 1.0), (1, 0.0), (2, 0.0)])
def test_completed_runs_are_verdicts(code, reward):
    require_code_verdict(TASK, reward, {"verifier_returncode": code, "resolved": code == 0})


@pytest.mark.parametrize("extra", [{}, {"model_patch": ""}, {"verifier_returncode": None}, {"verifier_returncode": -9}, {"verifier_returncode": 124},
                                   {"verifier_returncode": 125}, {"verifier_returncode": 126}, {"verifier_returncode": 127}, {"verifier_returncode": 137},
                                   {"verifier_returncode": True}, {"verifier_returncode": 1, "resolved": False, "error_category": "reward/testbed_corrupted"},
                                   {"verifier_returncode": 1, "resolved": False, "transport_error": True},
                                   {"verifier_returncode": 1, "resolved": False, "model_patch_error": "cannot read git"}])
def test_infrastructure_failures_never_become_zero_rewards(extra):
    with pytest.raises(RewardInfrastructureError):
        require_code_verdict(TASK, 0.0, extra)


@pytest.mark.parametrize("reward,extra", [(0.0, {"verifier_returncode": 0, "resolved": True}), (1.0, {"verifier_returncode": 1, "resolved": False}),
                                          (float("nan"), {"verifier_returncode": 0, "resolved": True}), (0.0, {"verifier_returncode": 1})])
def test_inconsistent_or_non_finite_records_are_rejected(reward, extra):
    with pytest.raises(RewardInfrastructureError):
        require_code_verdict(TASK, reward, extra)


def test_other_task_kinds_and_stop_classification():
    require_code_verdict({"dataset_type": "general_agent"}, 0.5, {})
    assert classify_stop("length", "partial candidate", None) == {"status": "limits_exceeded", "execute_tools": False, "keep_content": "partial candidate", "truncated": True}
    assert classify_stop("length", "", [{"name": "bash"}])["execute_tools"] is False          # half a command is not run
    assert classify_stop("stop", "done", [])["status"] == "idle" and classify_stop("tool_calls", None, [{"name": "bash"}]) == {
        "status": "continue", "execute_tools": True, "keep_content": "", "truncated": False}
    with pytest.raises(ValueError):
        classify_stop("content_filter", "", None)
