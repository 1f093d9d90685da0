"""The rule-table evaluator behind the science validators."""
from types import SimpleNamespace

import pytest

from archlab_b200.contracts import science_rules as sr


def _tree():
    return {"actor_rollout_ref": {"rollout": {"n": 4, "enforce_eager": True, "engine_kwargs": {"vllm": {"model_impl": "vllm"}},
                                              "custom": {"agent_framework": {"mask_unfinished_episode": False}}},
                                  "actor": {"megatron": {"dtype": "bfloat16"}, "optim": {"betas": (0.9, 0.95)}}},
            "data": {"truncation": "error"}}


def test_lookup_shorthands_and_optional_paths():
    e = SimpleNamespace(pilot=None, native_context=8)
    t = _tree()
    assert sr.lookup(t, e, "rollout.n") == 4 and sr.lookup(t, e, "mg.dtype") == "bfloat16"
    assert sr.lookup(t, e, "vllm") == {"model_impl": "vllm"} and sr.lookup(t, e, "agent.mask_unfinished_episode") is False
    assert sr.lookup(t, e, "e.native_context") == 8
    assert sr.lookup(t, e, "rollout.missing") is sr._ABSENT and sr.lookup(t, e, "rollout.missing?") is None
    assert sr.lookup(t, e, "pilot.step_limit") is sr._ABSENT


def test_requirements_literal_switch_and_function():
    e = SimpleNamespace(pilot=SimpleNamespace(step_limit=500), native_context=8)
    t = _tree()
    ok = sr.Rule("fine", {"rollout.n": sr.at_least(2), "rollout.enforce_eager": sr.ON, "agent.mask_unfinished_episode": sr.OFF,
                          "actor.optim.betas": [0.9, 0.95], "pilot.step_limit": 500, "data.truncation": "error"})
    assert ok.violated(e, t) is None
    assert sr.Rule("m", {"rollout.n": 8}).violated(e, t) == "rollout.n"
    assert sr.Rule("m", {"rollout.absent": sr.OFF}).violated(e, t) == "rollout.absent"          # a missing path never passes
    with pytest.raises(ValueError, match="^second$") as info:
        sr.check((ok, sr.Rule("skipped", {"rollout.n": 0}, lambda e: False), sr.Rule("second", {"data.truncation": "left"})), e, t)
    assert info.value.violated_path == "data.truncation"


def test_rule_messages_are_distinct_and_kwargs_conflicts_are_named():
    messages = [r.message for group in (sr.HEAD, sr.MUSE, sr.FAMILY, sr.CONVERSION, sr.COMMON) for r in group]
    assert len(messages) == len(set(messages)) and len(messages) >= 35
    t = _tree()
    t["actor_rollout_ref"]["rollout"]["engine_kwargs"]["vllm"].update(quantization="fp8", model="x")
    with pytest.raises(ValueError, match="override the serving contract: model, quantization"):
        sr.conversion_kwargs_conflict(SimpleNamespace(pilot=None), t)
