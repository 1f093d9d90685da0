"""Pipeline gate: a real (tiny) policy improves its reward under GRPO updates on its own rollouts."""
import torch

from archlab_b200.models import limite as L
from archlab_b200.train import grpo


def test_group_advantages_and_loss_contract():
    rewards = torch.tensor([1.0, 0.0, 0.0, 0.0, 1.0, 1.0])
    groups = torch.tensor([0, 0, 0, 1, 1, 2])
    try:
        grpo.group_advantages(rewards, groups)
        raise AssertionError("a single-rollout group must be refused")
    except ValueError:
        pass
    adv, info = grpo.group_advantages(rewards[:5], groups[:5])
    assert info.tolist() == [True] * 5 and abs(float(adv[:3].sum())) < 1e-5 and adv[0] > 0 > adv[1]
    adv2, info2 = grpo.group_advantages(torch.tensor([1.0, 1.0, 0.0, 1.0]), torch.tensor([0, 0, 1, 1]))
    assert info2.tolist() == [False, False, True, True] and adv2[:2].abs().sum() == 0
    old = torch.zeros(2, 3)
    new = torch.tensor([[0.0, 1.0, -1.0], [0.0, 0.0, 0.0]], requires_grad=True)      # ratios 1, e (> cap 2), 1/e
    loss, m = grpo.grpo_loss(new, old, torch.tensor([1.0, -1.0]), torch.ones(2, 3, dtype=torch.bool))
    loss.backward()
    assert new.grad[0, 1] == 0 and m["cap_fraction"] > 0 and new.grad[0, 0] < 0     # capped token: no gradient


def test_real_policy_grpo_update():
    torch.manual_seed(0)
    model = L.LimiteLM(L.LimiteConfig.tiny(vocab_size=16, num_hidden_layers=2))
    model.init_weights(0.1)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    target, P, G, n_prompts, n_roll = 7, 4, 6, 4, 8
    gen = torch.Generator().manual_seed(0)

    def rollouts():
        prompts = torch.randint(0, 16, (n_prompts, P), generator=gen).repeat_interleave(n_roll, 0)
        ids = prompts.clone()
        with torch.no_grad():
            for _ in range(G):
                nxt = torch.multinomial(model(ids)[:, -1].softmax(-1), 1, generator=gen)
                ids = torch.cat([ids, nxt], 1)
            old = grpo.sequence_logprobs(model, ids)
        mask = torch.zeros(ids.size(0), ids.size(1) - 1, dtype=torch.bool)
        mask[:, P - 1:] = True
        rewards = (ids[:, P:] == target).float().mean(1)          # reward: share of generated tokens equal to the target
        return {"ids": ids, "old_logp": old, "mask": mask, "rewards": rewards,
                "group_ids": torch.arange(n_prompts).repeat_interleave(n_roll), "policy_version": torch.zeros(ids.size(0))}

    first = float(rollouts()["rewards"].mean())
    for _ in range(40):
        metrics = grpo.grpo_step(model, opt, rollouts())
    last = float(rollouts()["rewards"].mean())
    assert last > first + 0.2 and 0 <= metrics["wasted_group_share"] <= 1 and metrics["cap_fraction"] == 0
