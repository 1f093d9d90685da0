"""When is a software-engineering reward a verdict, and when is it an accident of the infrastructure?

An executable verifier applies the hidden test patch after the rollout and runs the test command; exit code 0 means the
task is solved (reward 1), a small positive exit code means the tests ran and failed (reward 0).  Everything else is not
information about the policy: a verifier that never ran, was killed (negative codes, 137), timed out (124) or could not
start (125-127); a corrupted test bed; a transport failure between trainer and sandbox; a patch that could not be read.
Training on those as "reward 0" teaches the policy that infrastructure weather is its fault, so they raise
``RewardInfrastructureError`` and the group is dropped or retried.  The same goes for inconsistent records (reward 1
with failing tests, reward 0 with passing ones, non-finite rewards).

On the agent side: a response cut off by the context limit ends the episode as ``limits_exceeded`` (never as a normal
idle stop), its text is kept as it was produced, and a tool call that arrived in a truncated response is NOT executed
(its arguments may be half a command).  (Reference contracts: tests/test_mimo_reward_contract.py:17-60,
tests/test_mimo_truncation_contract.py:24-60 over the patched upstream runner.)
"""
from __future__ import annotations

import math

UNUSABLE_RETURN_CODES = frozenset({124, 125, 126, 127, 137})
CODE_DATASET = "opensource-code"


class RewardInfrastructureError(RuntimeError):
    """The reward says nothing about the policy; do not learn from it."""


def require_code_verdict(task: dict, reward: float, extra: dict) -> None:
    if task.get("dataset_type") != CODE_DATASET:
        return                                                     # other task kinds keep their own reward contracts
    code = extra.get("verifier_returncode")
    if type(code) is not int or code < 0 or code in UNUSABLE_RETURN_CODES:
        raise RewardInfrastructureError(f"the verifier did not complete (return code {code!r}) for {task.get('instance_id')}")
    for flag in ("transport_error", "model_patch_error"):
        if extra.get(flag):
            raise RewardInfrastructureError(f"{flag} for {task.get('instance_id')}: {extra[flag]}")
    if str(extra.get("error_category", "")).startswith("reward/"):
        raise RewardInfrastructureError(f"verifier infrastructure error {extra['error_category']} for {task.get('instance_id')}")
    if not isinstance(reward, (int, float)) or not math.isfinite(reward):
        raise RewardInfrastructureError("non-finite reward")
    resolved = extra.get("resolved")
    if type(resolved) is not bool or resolved != (code == 0) or float(reward) != (1.0 if resolved else 0.0):
        raise RewardInfrastructureError(f"inconsistent verdict for {task.get('instance_id')}: reward {reward}, code {code}, resolved {resolved!r}")


def classify_stop(finish_reason: str, content: str | None, tool_calls) -> dict:
    """What an agent loop does with one model response.  ``status``: ``continue`` (execute the tool call), ``idle`` (a normal
    final answer) or ``limits_exceeded``; ``execute_tools`` is False for a truncated response whatever it contains."""
    if finish_reason not in ("stop", "length", "tool_calls"):
        raise ValueError(f"unknown finish reason {finish_reason!r}")
    truncated = finish_reason == "length"
    calls = list(tool_calls or [])
    if truncated:
        status = "limits_exceeded"
    else:
        status = "continue" if calls else "idle"
    return {"status": status, "execute_tools": bool(calls) and not truncated, "keep_content": content or "", "truncated": truncated}
