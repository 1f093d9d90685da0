"""Agentic GRPO loop on CPU: the policy learns a rewarded token, tool observations are masked, stale groups are
dropped, and the evidence receipt passes the admission gate's learning-signal check."""
import json

import pytest
import torch

from archlab_b200.contracts.experiment import AgenticPilot
from archlab_b200.models.limite import LimiteConfig, LimiteLM
from archlab_b200.train import qualification as q
from archlab_b200.train import rl_loop as rl


def _model(seed=0):
    torch.manual_seed(seed)
    m = LimiteLM(LimiteConfig.tiny(vocab_size=32, num_hidden_layers=2))
    m.init_weights()
    return m


class EchoTool:
    """Token 5 is a tool call answered with two observation tokens; token 3 ends the episode."""

    def step(self, prompt, response):
        if response[-1] == 3:
            return "stop", []
        return "continue", ([9, 9] if response[-1] == 5 else [])


def test_policy_learns_the_rewarded_token_and_writes_evidence(tmp_path):
    model = _model()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    loop = rl.AgenticGRPO(model, opt, rl.ActorConfig(responses_per_prompt=8, max_new_tokens=4),
                          rl.LoopConfig(prompts_per_step=2, steps=25), verifier=lambda t: float(7 in t.tokens),
                          prompts=lambda i: (f"p{i}", [1, 2 + i % 3]), evidence_dir=tmp_path / "artifacts" / "run", seed=1)
    history = loop.run()
    early = sum(m["mean_reward"] for m in history[:5]) / 5
    late = sum(m["mean_reward"] for m in history[-5:]) / 5
    assert late > early + 0.3, (early, late)
    assert all(m["max_policy_lag"] == 0 for m in history) and loop.actor.version == loop.version == 25
    evidence = json.loads((tmp_path / "artifacts" / "run" / "pipeline-evidence.json").read_text())
    assert evidence["completed_verifiers"] == 25 * 2 * 8 and evidence["learner_steps"] == 25
    assert len(evidence["consumed_rollout_uids"]) == len(set(evidence["consumed_rollout_uids"])) == 400
    # a short run whose last update still has reward contrast passes the admission gate's learning-signal check
    model = _model(2)
    short = rl.AgenticGRPO(model, torch.optim.AdamW(model.parameters(), lr=1e-3), rl.ActorConfig(responses_per_prompt=8, max_new_tokens=4),
                           rl.LoopConfig(prompts_per_step=2, steps=3), verifier=lambda t: float(sum(t.tokens) % 2),
                           prompts=lambda i: (f"p{i}", [1, 2 + i % 3]), evidence_dir=tmp_path / "gate" / "artifacts" / "run", seed=4)
    short.run()
    verdict = q.check_learning_signal(tmp_path / "gate", AgenticPilot(minimum_tool_calls=0, minimum_observation_tokens=0,
                                                                      maximum_truncated_trajectories=10 ** 6))
    assert "status" not in verdict and verdict["observed"]["prompt_groups"] == 6 and verdict["grad_norm"] > 0


def test_tool_observations_are_masked_and_truncation_is_marked():
    model = _model(3)
    actor = rl.Actor(model, rl.ActorConfig(responses_per_prompt=16, max_new_tokens=5, max_context=64), EchoTool(), seed=5)
    group = actor.rollout_group("g", [1, 2])
    assert len({t.uid for t in group}) == 16
    for t in group:
        assert len(t.tokens) == len(t.policy_mask) == len(t.behaviour_logp)
        assert t.observation_tokens == 2 * t.tool_calls
        policy = [tok for tok, m in zip(t.tokens, t.policy_mask) if m]
        assert t.truncated == (len(policy) == 5 and policy[-1] != 3)
        assert all(lp <= 0 for lp in t.behaviour_logp)
        t.reward = float(len(policy))
    batch = rl.collate([group], "cpu")
    assert batch["ids"].shape[0] == 16 and batch["mask"].shape == batch["old_logp"].shape
    for r, t in enumerate(group):
        assert int(batch["mask"][r].sum()) == sum(t.policy_mask)              # observation tokens carry no gradient
        first = len(t.prompt) - 1
        assert not batch["mask"][r, :first].any()
    # the behaviour log-probabilities are those the learner recomputes for the same weights (ratio 1 at version 0)
    from archlab_b200.train.grpo import sequence_logprobs

    new = sequence_logprobs(model, batch["ids"])
    gap = ((new - batch["old_logp"]).abs() * batch["mask"]).max()
    assert gap < 1e-4, gap


def test_stale_groups_are_dropped_not_trained_on():
    queue = rl.ReplayQueue(max_policy_lag=1)
    mk = lambda v: [rl.Trajectory(uid=f"g{v}_{i}_{v}", prompt=[1], policy_version=v) for i in range(2)]
    for v in (0, 1, 2):
        queue.put(mk(v))
    taken = queue.take(3, learner_version=2)
    assert [g[0].policy_version for g in taken] == [1, 2] and queue.dropped_stale == 1 and len(queue) == 0


def test_contract_refusals():
    with pytest.raises(ValueError, match="multiple responses"):
        rl.ActorConfig(responses_per_prompt=1)
    with pytest.raises(ValueError, match="positive finite temperature"):
        rl.ActorConfig(temperature=0.0)
    model = _model()
    with pytest.raises(ValueError, match="temperature 1"):
        rl.AgenticGRPO(model, None, rl.ActorConfig(temperature=0.7), rl.LoopConfig(), lambda t: 0.0, lambda i: ("p", [1]))
    loop = rl.AgenticGRPO(model, torch.optim.SGD(model.parameters(), lr=0.1), rl.ActorConfig(responses_per_prompt=2, max_new_tokens=2),
                          rl.LoopConfig(steps=1), verifier=lambda t: float("nan"), prompts=lambda i: ("p", [1]))
    with pytest.raises(ValueError, match="non-finite reward"):
        loop.run()


def test_groups_without_a_verdict_are_counted_and_not_learned_from(tmp_path):
    import torch

    from archlab_b200.services.code_verdict import RewardInfrastructureError
    from archlab_b200.train import rl_loop as rl

    src = open(rl.__file__).read()
    assert "infrastructure_failed_groups" in src
    calls = {"n": 0}

    def verifier(t):
        calls["n"] += 1
        if t.uid.startswith("p1"):
            raise RewardInfrastructureError("sandbox timeout")
        return 1.0

    class Stub:
        def __init__(self):
            self.totals = {"completed_verifiers": 0, "tool_calls": 0, "masked_observation_tokens": 0, "truncated_trajectories": 0,
                           "reward_contrast_groups": 0, "wasted_groups": 0, "dropped_stale_groups": 0, "infrastructure_failed_groups": 0}
            self.next_prompt, self.verifier, self.put = 0, verifier, []
            self.prompts = lambda i: (f"p{i}", [1, 2])
            self.actor = type("A", (), {"rollout_group": staticmethod(lambda gid, prompt: [type("T", (), {"uid": f"{gid}-{k}", "tool_calls": 0, "observation_tokens": 0,
                                                                                                          "truncated": False, "reward": None})() for k in range(2)])})()
            self.queue = type("Q", (), {"put": lambda _self, g: self.put.append(g)})()

    stub = Stub()
    rl.AgenticGRPO.collect(stub, 3)
    assert stub.totals["infrastructure_failed_groups"] == 1 and len(stub.put) == 2 and stub.totals["completed_verifiers"] == 4
    assert all(t.reward == 1.0 for g in stub.put for t in g)
