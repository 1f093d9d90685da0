"""Admission of trajectories at the rollout boundary.

Behaviour contract (src/archlab/training/rollout.py:41-107; exercised by the reference's
tests/test_native_agentic_contract.py:82-92): a trajectory enters the learner only if its response
tokens, loss mask and behaviour log-probabilities line up one to one, the mask is exactly the union of
the generated spans (tool observations are unmasked and carry log-probability 0), the engine reported the
span of policy versions that produced it, and it ended for a named reason.  What comes back is the
per-response record the learner logs (`RolloutMetadata`).

The checks are a table of (name, predicate) pairs evaluated over one normalised view of the trajectory,
so a refusal names the rule that failed and a new rule is one more row.
"""
from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable

TERMINATIONS = ("completed", "truncated")


class InadmissibleTrajectory(ValueError):
    def __init__(self, rule: str, detail: str):
        super().__init__(f"{rule}: {detail}")
        self.rule = rule


@dataclass(frozen=True)
class RolloutMetadata:
    question_id: str
    group_id: str
    response_id: str
    session_id: int
    policy_version_first: int
    policy_version_last: int
    termination_reason: str
    rng_identity: str
    rng_replayable: bool          # identity only: an asynchronous engine is not bit-replayable from a seed
    generated_tokens: int
    observation_tokens: int
    native_eos_tokens: int
    terminal_native_eos: bool
    context_limit_reached: bool


def _field(obj: Any, name: str, default=None):
    """Trajectories arrive as objects (the engine's dataclass) or as plain mappings (replayed JSON)."""
    if isinstance(obj, dict):
        return obj.get(name, default)
    return getattr(obj, name, default)


def _is_count(x) -> bool:
    return type(x) is int and x >= 0


@dataclass
class _View:
    """Everything the rules look at, pulled out of the trajectory once."""
    prompt: list
    response: list
    mask: list
    logprobs: list | None
    spans: list
    versions: tuple
    termination: Any
    context: int
    span_mask: list = field(default_factory=list)
    spans_ordered: bool = True

    @classmethod
    def of(cls, traj, context: int) -> "_View":
        extra = _field(traj, "extra_fields", {}) or {}
        reward = _field(traj, "reward_info", {}) or {}
        v = cls(list(_field(traj, "prompt_ids", []) or []), list(_field(traj, "response_ids", []) or []),
                list(_field(traj, "response_mask", []) or []), _field(traj, "response_logprobs"),
                [tuple(s) for s in (_field(traj, "generation_spans", []) or [])],
                (extra.get("min_global_steps"), extra.get("max_global_steps")), reward.get("termination_kind"), context)
        # the mask the spans imply; spans must be disjoint, non-empty, ascending and inside the response
        cover, cursor = [0] * len(v.response), 0
        for lo, hi in v.spans:
            if not (type(lo) is int and type(hi) is int and cursor <= lo < hi <= len(v.response)):
                v.spans_ordered = False
                break
            cover[lo:hi] = [1] * (hi - lo)
            cursor = hi
        v.span_mask = cover
        return v


_RULES: tuple[tuple[str, Callable[[_View], bool], str], ...] = (
    ("non-empty", lambda v: bool(v.prompt) and bool(v.response), "prompt and response must both hold tokens"),
    ("context", lambda v: len(v.prompt) + len(v.response) <= v.context, "prompt + response exceed the context"),
    ("token-ids", lambda v: all(_is_count(t) for t in v.prompt) and all(_is_count(t) for t in v.response),
     "token ids must be non-negative integers"),
    ("alignment", lambda v: v.logprobs is not None and len(v.response) == len(v.mask) == len(v.logprobs),
     "response tokens, loss mask and behaviour log-probabilities must have one entry per token"),
    ("span-order", lambda v: v.spans_ordered, "generation spans overlap, are empty or are out of order"),
    ("span-mask", lambda v: any(v.span_mask) and v.mask == v.span_mask,
     "the loss mask must select exactly the generated spans"),
    ("logprobs", lambda v: all(math.isfinite(p) and (m or p == 0) for p, m in zip(v.logprobs, v.mask)),
     "behaviour log-probabilities must be finite, and zero on tool observations"),
    ("policy-versions", lambda v: all(_is_count(x) for x in v.versions) and v.versions[0] <= v.versions[1],
     "the engine must report min_global_steps <= max_global_steps"),
    ("termination", lambda v: v.termination in TERMINATIONS, f"termination_kind must be one of {TERMINATIONS}"),
)


def validate_trajectory(trajectory, *, question_id: str, group_id: str, response_id: str, session_id: int, context: int,
                        eos_ids: Iterable[int], rng_identity: str) -> RolloutMetadata:
    names = {"question_id": question_id, "group_id": group_id, "response_id": response_id, "rng_identity": rng_identity}
    blank = [k for k, s in names.items() if not (isinstance(s, str) and s)]
    if blank:
        raise InadmissibleTrajectory("identity", f"missing {', '.join(blank)}")
    if not _is_count(session_id):
        raise InadmissibleTrajectory("identity", "session id must be a non-negative integer")
    view = _View.of(trajectory, int(context))
    for rule, holds, detail in _RULES:
        if not holds(view):
            raise InadmissibleTrajectory(rule, detail)
    eos = set(eos_ids)
    generated = [t for t, m in zip(view.response, view.mask) if m]
    return RolloutMetadata(
        question_id=question_id, group_id=group_id, response_id=response_id, session_id=session_id,
        policy_version_first=view.versions[0], policy_version_last=view.versions[1], termination_reason=view.termination,
        rng_identity=rng_identity, rng_replayable=False, generated_tokens=len(generated),
        observation_tokens=len(view.response) - len(generated), native_eos_tokens=sum(t in eos for t in generated),
        terminal_native_eos=generated[-1] in eos, context_limit_reached=len(view.prompt) + len(view.response) == view.context)


def _dig(config, path: str, default=None):
    """``a.b.c`` lookup through attribute- or key-addressed configuration nodes."""
    node = config
    for part in path.split("."):
        if node is None:
            return default
        if isinstance(node, dict):
            node = node.get(part)
        elif hasattr(node, part):
            node = getattr(node, part)
        elif hasattr(node, "get"):
            node = node.get(part)
        else:
            return default
    return default if node is None else node


class RolloutContract:
    """Boundary callback shared by every rollout backend: built once from the composed trainer configuration,
    called per finished trajectory, returns the metadata record as a plain dict."""

    def __init__(self, config):
        model_dir = Path(_dig(config, "actor_rollout_ref.model.path"))
        eos = json.loads((model_dir / "generation_config.json").read_text())["eos_token_id"]
        self.eos_ids = frozenset([eos] if isinstance(eos, int) else eos)
        if not self.eos_ids or not all(_is_count(t) for t in self.eos_ids):
            raise ValueError("generation_config.json does not name a valid end-of-sequence token")
        self.context = int(_dig(config, "actor_rollout_ref.rollout.max_model_len"))
        engine, seed = _dig(config, "actor_rollout_ref.rollout.name"), _dig(config, "actor_rollout_ref.rollout.seed")
        self.rng_scope = f"{engine}:engine-seed={seed}:backend-managed"
        self.mask_unfinished = bool(
            _dig(config, "actor_rollout_ref.rollout.custom.agent_framework.mask_unfinished_episode", False))

    def __call__(self, *, trajectory, sample_fields, group_id, response_id, session_id) -> dict:
        meta = validate_trajectory(
            trajectory, question_id=sample_fields["extra_info"]["instance_id"], group_id=group_id, response_id=response_id,
            session_id=session_id, context=self.context, eos_ids=self.eos_ids, rng_identity=f"{self.rng_scope}:{response_id}")
        if self.mask_unfinished:
            finished = (_field(trajectory, "reward_info", {}) or {}).get("finished")
            if finished is not (meta.termination_reason == "completed"):
                raise InadmissibleTrajectory("finished-flag", "the agent must set `finished` to match the termination "
                                                              "before unfinished episodes are masked")
        return asdict(meta)
