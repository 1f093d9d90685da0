"""Trajectory admission (behaviour of the reference's tests/test_native_agentic_contract.py:82-92 and of
src/archlab/training/rollout.py): aligned tokens / mask / log-probabilities, mask = generated spans, zero
log-probability on tool observations, reported policy versions, named termination."""
import json
from types import SimpleNamespace

import pytest

from archlab_b200.train.rollout import InadmissibleTrajectory, RolloutContract, validate_trajectory


def _traj(**over):
    base = dict(prompt_ids=[5, 6, 7], response_ids=[10, 11, 2, 40, 41, 12, 2], response_mask=[1, 1, 1, 0, 0, 1, 1],
                response_logprobs=[-0.1, -0.2, -0.3, 0.0, 0.0, -0.4, -0.5], generation_spans=[(0, 3), (5, 7)],
                extra_fields={"min_global_steps": 1, "max_global_steps": 2}, reward_info={"termination_kind": "completed"})
    base.update(over)
    return SimpleNamespace(**base)


ID = dict(question_id="task", group_id="group", response_id="group_0_0", session_id=0, context=64, eos_ids={2},
          rng_identity="recorded-fixture")


def test_admitted_trajectory_yields_the_learner_record():
    m = validate_trajectory(_traj(), **ID)
    assert (m.policy_version_first, m.policy_version_last) == (1, 2)
    assert (m.generated_tokens, m.observation_tokens, m.native_eos_tokens) == (5, 2, 2)
    assert m.terminal_native_eos and not m.context_limit_reached and not m.rng_replayable
    assert validate_trajectory(_traj(), **{**ID, "context": 10}).context_limit_reached
    # a replayed JSON record (plain mapping) is admitted the same way
    assert validate_trajectory(vars(_traj()), **ID) == m


@pytest.mark.parametrize("rule,change", [
    ("non-empty", dict(response_ids=[], response_mask=[], response_logprobs=[], generation_spans=[])),
    ("context", dict(prompt_ids=list(range(60)))),
    ("token-ids", dict(prompt_ids=[5, -1, 7])),
    ("alignment", dict(response_logprobs=None)),
    ("alignment", dict(response_mask=[1, 1, 1, 0, 0, 1])),
    ("span-order", dict(generation_spans=[(5, 7), (0, 3)])),
    ("span-order", dict(generation_spans=[(0, 3), (2, 7)])),
    ("span-mask", dict(response_mask=[1, 1, 1, 1, 0, 1, 1])),
    ("span-mask", dict(generation_spans=[], response_mask=[0] * 7, response_logprobs=[0.0] * 7)),
    ("logprobs", dict(response_logprobs=[-0.1, -0.2, -0.3, -0.9, 0.0, -0.4, -0.5])),
    ("logprobs", dict(response_logprobs=[-0.1, float("nan"), -0.3, 0.0, 0.0, -0.4, -0.5])),
    ("policy-versions", dict(extra_fields={"min_global_steps": 3, "max_global_steps": 2})),
    ("policy-versions", dict(extra_fields={})),
    ("termination", dict(reward_info={"termination_kind": "crashed"})),
])
def test_each_rule_refuses_with_its_name(rule, change):
    with pytest.raises(InadmissibleTrajectory) as err:
        validate_trajectory(_traj(**change), **ID)
    assert err.value.rule == rule and isinstance(err.value, ValueError)


def test_identity_is_required():
    for bad in (dict(question_id=""), dict(rng_identity=None), dict(session_id=-1), dict(session_id=True)):
        with pytest.raises(InadmissibleTrajectory) as err:
            validate_trajectory(_traj(), **{**ID, **bad})
        assert err.value.rule == "identity"


def test_contract_object_reads_the_composed_configuration(tmp_path):
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [2, 9]}))
    rollout = {"name": "vllm", "seed": 7, "max_model_len": 64,
               "custom": {"agent_framework": {"mask_unfinished_episode": True}}}
    cfg = {"actor_rollout_ref": {"model": {"path": str(tmp_path)}, "rollout": rollout}}
    contract = RolloutContract(cfg)
    fields = {"extra_info": {"instance_id": "task"}}
    call = dict(sample_fields=fields, group_id="g", response_id="g_0", session_id=1)
    done = _traj(reward_info={"termination_kind": "completed", "finished": True})
    rec = contract(trajectory=done, **call)
    assert rec["rng_identity"] == "vllm:engine-seed=7:backend-managed:g_0" and rec["native_eos_tokens"] == 2
    with pytest.raises(InadmissibleTrajectory) as err:
        contract(trajectory=_traj(reward_info={"termination_kind": "truncated", "finished": True}), **call)
    assert err.value.rule == "finished-flag"
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": []}))
    with pytest.raises(ValueError):
        RolloutContract(cfg)
