"""Adapter warm-up -> full-weight training: two clocks, fp32 masters, optimizer history carried across the switch."""
import math

import pytest
import torch

from archlab_b200.optim.split_adamw import FORMAT, MasterAdamW, SplitAdamW, build_warmup_optimizer, warmup_learning_rates

SCHEDULE = {"target_tokens": 1000, "full_weight_start_step": 10, "full_weight_start_tokens": 400, "adapter_peak_lr": 1e-3, "adapter_warmup_steps": 5,
            "backbone_peak_lr": 1e-4, "backbone_warmup_steps": 4}


def test_two_clocks():
    a, b = warmup_learning_rates(10, 400, SCHEDULE)
    assert a == pytest.approx(1e-3 * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.4)))) and b == pytest.approx(1e-4 * 0.25 * 1.0)
    a_end, b_end = warmup_learning_rates(40, 1000, SCHEDULE)
    assert a_end == pytest.approx(1e-4) and b_end == pytest.approx(1e-5)                      # both end at 10 % of their peaks
    assert warmup_learning_rates(2, 100, SCHEDULE)[0] == pytest.approx(1e-3 * 0.6 * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.1))))


def test_master_weights_accumulate_updates_that_bf16_would_lose():
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.ones(64, dtype=torch.bfloat16))
    opt = MasterAdamW([p], lr=1e-4, betas=(0.9, 0.95))
    for _ in range(30):
        p.grad = torch.ones_like(p)
        opt.step()
    master = opt.state[p]["master"]
    assert master.dtype == torch.float32 and float(master[0]) == pytest.approx(1 - 30 * 1e-4, rel=1e-3)
    assert torch.equal(p.detach(), master.bfloat16())                                           # 1 - 1e-4 alone would round back to 1 in bf16
    q = torch.nn.Parameter(torch.ones(4))
    ref = torch.nn.Parameter(torch.ones(4))
    mine, theirs = MasterAdamW([q], lr=1e-2, weight_decay=0.1), torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for i in range(5):
        q.grad = ref.grad = torch.full((4,), float(i + 1))
        mine.step(), theirs.step()
    assert torch.allclose(q, ref, atol=1e-6) and mine.state[q]["master"] is None


def test_history_survives_the_switch():
    torch.manual_seed(1)
    adapter, backbone = torch.nn.Linear(4, 4), torch.nn.Linear(4, 4).bfloat16()
    for p in backbone.parameters():
        p.requires_grad_(False)
    phase1 = build_warmup_optimizer(adapter.parameters(), backbone.parameters())
    assert isinstance(phase1, torch.optim.AdamW)
    for _ in range(3):
        adapter(torch.randn(2, 4)).sum().backward()
        phase1.step(), phase1.zero_grad()
    saved = phase1.state_dict()
    for p in backbone.parameters():
        p.requires_grad_(True)
    phase2 = build_warmup_optimizer(adapter.parameters(), backbone.parameters())
    assert isinstance(phase2, SplitAdamW) and len(phase2.param_groups) == 2
    phase2.load_state_dict(saved)                                                               # phase-1 state: adapter half only
    assert int(phase2.adapter.state[adapter.weight]["step"]) == 3 and not phase2.backbone.state
    phase2.set_learning_rates(*warmup_learning_rates(10, 400, SCHEDULE))
    assert phase2.backbone.param_groups[0]["lr"] == pytest.approx(2.5e-5)
    backbone(adapter(torch.randn(2, 4)).bfloat16()).float().sum().backward()
    phase2.step(), phase2.zero_grad()
    state = phase2.state_dict()
    assert state["format"] == FORMAT and int(phase2.adapter.state[adapter.weight]["step"]) == 4
    again = build_warmup_optimizer(adapter.parameters(), backbone.parameters())
    again.load_state_dict(state)
    assert torch.equal(again.backbone.state[backbone.weight]["master"], phase2.backbone.state[backbone.weight]["master"])
    with pytest.raises(ValueError, match="unsupported"):
        again.load_state_dict({"format": "other"})
