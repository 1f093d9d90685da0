"""Distillation stages on a toy teacher / student: schedules, curriculum, latent matching, chunked KL
gradients (against the unchunked computation), on-policy rollout, checkpoint fingerprinting."""
import math

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from archlab_b200.train import distill as D


class Mixer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.f = nn.Linear(c, c)

    def forward(self, hidden_states, scale=1.0):
        return self.f(hidden_states) * scale


class Toy(nn.Module):
    def __init__(self, V=17, C=8, L=3, seed=0):
        super().__init__()
        torch.manual_seed(seed)
        self.emb = nn.Embedding(V, C)
        self.mix = nn.ModuleList(Mixer(C) for _ in range(L))
        self.head = nn.Linear(C, V)

    def hidden(self, ids):
        h = self.emb(ids)
        for m in self.mix:
            h = h + torch.tanh(m(h, scale=0.5))
        return h

    def forward(self, ids):
        return self.head(self.hidden(ids))


def test_schedules_and_curriculum():
    assert D.wsd_lr(1, 1000, 1.0) == pytest.approx(1 / 30)
    assert D.wsd_lr(500, 1000, 1.0) == 1.0 and D.wsd_lr(1000, 1000, 1.0) == pytest.approx(0.1)
    assert D.cosine_lr(0, 100, 1.0, 0.1, 0.1) == pytest.approx(0.1) and D.cosine_lr(99, 100, 1.0, 0.1, 0.1) == pytest.approx(0.1)
    with pytest.raises(ValueError):
        D.wsd_lr(1, 0, 1.0)
    assert D.horizons(4, 32) == (4, 8, 16, 32)
    with pytest.raises(ValueError):
        D.horizons(4, 24)
    cur = D.HorizonCurriculum(4)
    grew = [cur.update(1.0, max_gen_tokens=16, plateau_steps=3) for _ in range(5)]
    assert grew == [False, False, False, True, False] and cur.gen_tokens == 8 and cur.phase == 1
    div = D.HorizonCurriculum(4)
    assert not any(div.update(1.0 + 0.2 * i, max_gen_tokens=16, plateau_steps=3) for i in range(8))   # diverging: no growth
    with pytest.raises(FloatingPointError):
        cur.update(math.nan, max_gen_tokens=16)


def test_latent_matching_fits_each_layer():
    teacher = Toy(seed=0)
    switches = {1: Mixer(8), 2: Mixer(8)}
    mixers = {1: teacher.mix[1], 2: teacher.mix[2]}
    opt = torch.optim.Adam([p for s in switches.values() for p in s.parameters()], lr=3e-2)
    ids = torch.randint(0, 17, (4, 12))
    first = D.latent_match_step(teacher, mixers, switches, opt, ids)
    for _ in range(150):
        last = D.latent_match_step(teacher, mixers, switches, opt, ids)
    assert last["loss"] < 0.05 * first["loss"] and set(last["per_layer"]) == {1, 2}
    with pytest.raises(ValueError):
        D.latent_match_step(teacher, {1: teacher.mix[1]}, switches, opt, ids)


@pytest.mark.parametrize("direction", ["forward", "reverse"])
def test_chunked_kl_matches_full_gradient(direction):
    teacher, student, ref = Toy(seed=0), Toy(seed=1), Toy(seed=1)
    ids = torch.randint(0, 17, (3, 10))
    mask = torch.rand(3, 10) > 0.3
    val = D.chunked_kl_step(teacher.hidden, student.hidden, teacher.head, student.head, ids, mask, direction=direction, chunk_tokens=7)
    tl, sl = teacher(ids).detach(), ref(ids)
    kl = D._kl_rows(tl, sl) if direction == "forward" else D._kl_rows(sl, tl)
    full = (kl * mask).sum() / mask.sum()
    full.backward()
    assert val == pytest.approx(float(full), rel=1e-5)
    for a, b in zip(student.parameters(), ref.parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-6)


def test_rollout_mask_and_two_timescales(tmp_path):
    student = Toy(seed=2)
    g = torch.Generator().manual_seed(0)
    ids, mask = D.rollout(student, torch.randint(0, 17, (2, 5)), 4, generator=g)
    assert ids.shape == (2, 9) and mask[:, 4:8].all() and mask.sum() == 8
    switches = {0: student.mix[0]}
    opt = D.two_timescale_optimizer(student, switches, lr=1e-3, backbone_lr_ratio=0.1)
    assert {gr["role"]: gr["lr"] for gr in opt.param_groups} == {"switch": 1e-3, "backbone": 1e-4}
    fp = D.contract_hash({"stage": 2, "seed": 0})
    path = D.save_stage_checkpoint(tmp_path, 3, {"student": student}, opt, [D.rank_rng_state()], fp, {"tokens": 99})
    other = Toy(seed=5)
    opt2 = D.two_timescale_optimizer(other, {0: other.mix[0]}, lr=1e-3, backbone_lr_ratio=0.1)
    info = D.load_stage_checkpoint(path, {"student": other}, opt2, fp)
    assert info == {"step": 3, "extra": {"tokens": 99}} and torch.equal(other.head.weight, student.head.weight)
    with pytest.raises(ValueError):
        D.load_stage_checkpoint(path, {"student": other}, opt2, D.contract_hash({"stage": 3}))
    with pytest.raises(ValueError):
        D.load_stage_checkpoint(path, {"student": other}, opt2, fp, world=2)
