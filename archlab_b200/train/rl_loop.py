"""Agentic GRPO loop: actor (multi-turn rollouts with tools) -> verifier -> bounded replay -> learner step -> weight sync.

One process, colocated: the learner's model and the actor's copy live on the same device and the actor is refreshed by a
full-weight copy every ``sync_every`` learner steps (the "naive" full-weight synchronisation the experiment validators
pin).  The pieces and the rules they keep (what the reference's RL launcher enforces through its trainer tree:
src/archlab/training/config.py:149-229, rollout.py:17-247, qualification.py:360-420):

* **Actor**: ``n`` responses per prompt sampled at a positive temperature with full support (no top-k / top-p); every
  policy token records its behaviour log-probability and the policy version that produced it.  A tool environment may
  answer a tool call with observation tokens: they enter the context but are *masked* (no gradient, no behaviour
  probability).  A response that hits the turn or the context limit is marked truncated and stays in its group
  (unfinished trajectories remain visible; their reward is whatever the verifier gives the partial text).
* **Replay**: groups wait in a queue until a learner step takes them; a group whose policy version lags the learner by
  more than ``max_policy_lag`` steps is dropped and counted, never trained on.
* **Learner**: group-centred advantages, clipped importance ratio with the hard cap of 2, no KL term
  (``train.grpo``); groups without reward contrast give no gradient and are reported as wasted.
* **Evidence**: after every learner step the loop rewrites ``pipeline-evidence.json`` atomically with the counters the
  admission gate reads (completed verifiers, tool calls, masked observation tokens, truncated trajectories, groups with
  reward contrast, gradient norm, the uids of the rollouts the update consumed).
"""
from __future__ import annotations

import copy
import json
import math
from collections import deque
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Protocol

import torch

from ..contracts.substrate import atomic_write_json
from ..services.code_verdict import RewardInfrastructureError
from .grpo import GRPOConfig, grpo_step


class ToolEnvironment(Protocol):
    """Decides, after each policy token, whether the episode goes on."""

    def step(self, prompt: list[int], response: list[int]) -> tuple[str, list[int]]:
        """-> ("continue" | "stop", observation tokens appended to the context when a tool was called)."""


class NoTools:
    def __init__(self, eos: int | None = None):
        self.eos = eos

    def step(self, prompt, response):
        return ("stop" if self.eos is not None and response and response[-1] == self.eos else "continue"), []


@dataclass
class Trajectory:
    uid: str
    prompt: list[int]
    tokens: list[int] = field(default_factory=list)          # everything after the prompt: policy and observation tokens
    policy_mask: list[bool] = field(default_factory=list)    # True where the policy chose the token
    behaviour_logp: list[float] = field(default_factory=list)
    policy_version: int = 0
    tool_calls: int = 0
    truncated: bool = False
    reward: float | None = None

    @property
    def observation_tokens(self) -> int:
        return sum(1 for m in self.policy_mask if not m)


@dataclass(frozen=True)
class ActorConfig:
    responses_per_prompt: int = 4
    max_new_tokens: int = 16
    max_context: int = 128
    temperature: float = 1.0

    def __post_init__(self):
        if self.responses_per_prompt < 2:
            raise ValueError("GRPO requires multiple responses per prompt")
        if not (isinstance(self.temperature, (int, float)) and math.isfinite(self.temperature) and self.temperature > 0):
            raise ValueError("behaviour sampling needs a positive finite temperature")


class Actor:
    def __init__(self, model, cfg: ActorConfig, environment: ToolEnvironment | None = None, *, seed: int = 0):
        self.model, self.cfg, self.env = model, cfg, environment or NoTools()
        dev = next(model.parameters()).device
        self.gen = torch.Generator(device=dev).manual_seed(seed)
        self.version = 0

    def load_weights(self, state: dict, version: int) -> None:
        self.model.load_state_dict(state)
        self.version = version

    @torch.no_grad()
    def rollout_group(self, group_id: str, prompt: list[int]) -> list[Trajectory]:
        """``responses_per_prompt`` episodes of one prompt, advanced together one token at a time."""
        cfg = self.cfg
        dev = next(self.model.parameters()).device
        group = [Trajectory(uid=f"{group_id}_{i}_{self.version}", prompt=list(prompt), policy_version=self.version)
                 for i in range(cfg.responses_per_prompt)]
        live = list(range(len(group)))
        was_training = self.model.training
        self.model.eval()
        while live:
            width = max(len(group[i].prompt) + len(group[i].tokens) for i in live)
            rows = []
            for i in live:                                        # left-pad with the first prompt token (causal: harmless)
                ctx = group[i].prompt + group[i].tokens
                rows.append([ctx[0]] * (width - len(ctx)) + ctx)
            logits = self.model(torch.tensor(rows, device=dev))[:, -1, :].float() / cfg.temperature
            logp = logits.log_softmax(-1)
            choice = torch.multinomial(logp.exp(), 1, generator=self.gen)[:, 0]
            taken = logp.gather(1, choice[:, None])[:, 0].tolist()
            still = []
            for slot, i in enumerate(live):
                t = group[i]
                t.tokens.append(int(choice[slot]))
                t.policy_mask.append(True)
                t.behaviour_logp.append(taken[slot])
                policy_part = [tok for tok, m in zip(t.tokens, t.policy_mask) if m]
                verdict, observation = self.env.step(t.prompt, policy_part)
                if observation:
                    t.tool_calls += 1
                    t.tokens += list(observation)
                    t.policy_mask += [False] * len(observation)
                    t.behaviour_logp += [0.0] * len(observation)
                n_policy = sum(t.policy_mask)
                if verdict == "stop":
                    continue
                if n_policy >= cfg.max_new_tokens or len(t.prompt) + len(t.tokens) >= cfg.max_context:
                    t.truncated = True
                    continue
                still.append(i)
            live = still
        self.model.train(was_training)
        return group


class ReplayQueue:
    """Groups between actor and learner; enforces the policy-lag bound."""

    def __init__(self, max_policy_lag: int):
        if max_policy_lag < 0:
            raise ValueError("policy lag bound must be non-negative")
        self.max_lag = max_policy_lag
        self.groups: deque[list[Trajectory]] = deque()
        self.dropped_stale = 0

    def put(self, group: list[Trajectory]) -> None:
        self.groups.append(group)

    def take(self, count: int, learner_version: int) -> list[list[Trajectory]]:
        out = []
        while self.groups and len(out) < count:
            g = self.groups.popleft()
            if learner_version - min(t.policy_version for t in g) > self.max_lag:
                self.dropped_stale += 1
                continue
            out.append(g)
        return out

    def __len__(self):
        return len(self.groups)


def collate(groups: list[list[Trajectory]], device) -> dict:
    """Right-padded batch for ``grpo_step``: ids [N, T], old_logp / mask [N, T - 1] aligned with next-token positions."""
    rows = [t for g in groups for t in g]
    width = max(len(t.prompt) + len(t.tokens) for t in rows)
    ids = torch.zeros(len(rows), width, dtype=torch.long)
    old = torch.zeros(len(rows), width - 1)
    mask = torch.zeros(len(rows), width - 1, dtype=torch.bool)
    for r, t in enumerate(rows):
        seq = t.prompt + t.tokens
        ids[r, :len(seq)] = torch.tensor(seq)
        ids[r, len(seq):] = seq[-1]
        first = len(t.prompt) - 1                                  # position whose next token is the first response token
        old[r, first:first + len(t.tokens)] = torch.tensor(t.behaviour_logp)
        mask[r, first:first + len(t.tokens)] = torch.tensor(t.policy_mask)
    group_ids = torch.tensor([gi for gi, g in enumerate(groups) for _ in g])
    rewards = torch.tensor([float(t.reward) for t in rows])
    return {"ids": ids.to(device), "old_logp": old.to(device), "mask": mask.to(device), "rewards": rewards.to(device),
            "group_ids": group_ids.to(device), "policy_version": torch.tensor([t.policy_version for t in rows])}


@dataclass
class LoopConfig:
    prompts_per_step: int = 2
    max_policy_lag: int = 1
    sync_every: int = 1
    steps: int = 4
    grpo: GRPOConfig = field(default_factory=GRPOConfig)


class AgenticGRPO:
    def __init__(self, learner, optimizer, actor_cfg: ActorConfig, loop: LoopConfig, verifier: Callable[[Trajectory], float],
                 prompts: Callable[[int], tuple[str, list[int]]], *, environment: ToolEnvironment | None = None,
                 evidence_dir=None, seed: int = 0):
        if actor_cfg.temperature != 1.0:
            # the learner evaluates log-probabilities of the unscaled distribution; a tempered behaviour policy would
            # make every importance ratio wrong
            raise ValueError("the learner's log-probabilities are taken at temperature 1: sample at temperature 1")
        self.learner, self.optimizer, self.loop, self.verifier, self.prompts = learner, optimizer, loop, verifier, prompts
        self.actor = Actor(copy.deepcopy(learner), actor_cfg, environment, seed=seed)
        self.queue = ReplayQueue(loop.max_policy_lag)
        self.version = 0
        self.next_prompt = 0
        self.evidence_dir = Path(evidence_dir) if evidence_dir is not None else None
        self.totals = {"completed_verifiers": 0, "tool_calls": 0, "masked_observation_tokens": 0, "truncated_trajectories": 0,
                       "reward_contrast_groups": 0, "wasted_groups": 0, "dropped_stale_groups": 0, "infrastructure_failed_groups": 0}
        self.history: list[dict] = []

    def collect(self, groups: int) -> None:
        for _ in range(groups):
            group_id, prompt = self.prompts(self.next_prompt)
            self.next_prompt += 1
            group = self.actor.rollout_group(group_id, prompt)
            try:
                rewards = [float(self.verifier(t)) for t in group]
            except RewardInfrastructureError:
                # the verifier did not reach a verdict for some member: nothing of the group is learned from (a group with a
                # member missing would shift its own baseline), and the failure is counted, not hidden as a zero reward
                self.totals["infrastructure_failed_groups"] += 1
                continue
            for t, reward in zip(group, rewards):
                t.reward = reward
                if not math.isfinite(t.reward):
                    raise ValueError(f"verifier returned a non-finite reward for {t.uid}")
                self.totals["completed_verifiers"] += 1
                self.totals["tool_calls"] += t.tool_calls
                self.totals["masked_observation_tokens"] += t.observation_tokens
                self.totals["truncated_trajectories"] += int(t.truncated)
            self.queue.put(group)

    def learn(self) -> dict:
        groups = self.queue.take(self.loop.prompts_per_step, self.version)
        self.totals["dropped_stale_groups"] = self.queue.dropped_stale
        if not groups:
            return {"skipped": "no admissible groups"}
        contrast = sum(1 for g in groups if len({t.reward for t in g}) > 1)
        self.totals["reward_contrast_groups"] += contrast
        self.totals["wasted_groups"] += len(groups) - contrast
        device = next(self.learner.parameters()).device
        metrics = grpo_step(self.learner, self.optimizer, collate(groups, device), self.loop.grpo)
        self.version += 1
        if self.version % self.loop.sync_every == 0:
            self.actor.load_weights(self.learner.state_dict(), self.version)         # full-weight synchronisation
        metrics.update(step=self.version, groups=len(groups), reward_contrast_groups=contrast,
                       mean_reward=sum(t.reward for g in groups for t in g) / sum(len(g) for g in groups),
                       consumed_rollout_uids=[t.uid for g in groups for t in g],
                       max_policy_lag=max(self.version - 1 - t.policy_version for g in groups for t in g))
        self.history.append(metrics)
        self._write_evidence(metrics)
        return metrics

    def _write_evidence(self, last: dict) -> None:
        if self.evidence_dir is None:
            return
        consumed = [uid for m in self.history for uid in m["consumed_rollout_uids"]]
        atomic_write_json(self.evidence_dir / "pipeline-evidence.json", {
            **{k: self.totals[k] for k in ("completed_verifiers", "tool_calls", "masked_observation_tokens", "truncated_trajectories",
                                           "reward_contrast_groups")},
            "grad_norm": last["grad_norm"], "loss": last["loss"], "learner_steps": self.version, "consumed_rollout_uids": consumed,
            "dropped_stale_groups": self.totals["dropped_stale_groups"], "wasted_groups": self.totals["wasted_groups"],
            "infrastructure_failed_groups": self.totals["infrastructure_failed_groups"]})

    def run(self) -> list[dict]:
        for _ in range(self.loop.steps):
            self.collect(self.loop.prompts_per_step)
            self.learn()
        return self.history


def main(argv=None) -> int:
    """Smoke loop on a tiny Limite model: reward 1 for responses that contain a target token (synthetic task)."""
    import argparse

    from ..models.limite import LimiteConfig, LimiteLM

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--target-token", type=int, default=7)
    ap.add_argument("--evidence-dir", default=None)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    torch.manual_seed(a.seed)
    model = LimiteLM(LimiteConfig.tiny())
    model.init_weights() if hasattr(model, "init_weights") else None
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    loop = AgenticGRPO(model, opt, ActorConfig(responses_per_prompt=4, max_new_tokens=6), LoopConfig(steps=a.steps),
                       verifier=lambda t: float(a.target_token in t.tokens), prompts=lambda i: (f"p{i}", [1, 2 + i % 3]),
                       evidence_dir=a.evidence_dir, seed=a.seed)
    for m in loop.run():
        print(json.dumps({k: v for k, v in m.items() if k != "consumed_rollout_uids"}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
