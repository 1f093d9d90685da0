"""The three distillation stages as chained, resumable runs on a toy teacher / student."""
import copy
import json

import pytest
import torch
import torch.nn as nn

from archlab_b200.train import distill_stages as S
from tests.test_distill_cpu import Mixer, Toy


class Switch(nn.Module):
    """Replacement mixer: a different parameterisation of the same signature."""

    def __init__(self, c):
        super().__init__()
        self.a, self.b = nn.Linear(c, c, bias=False), nn.Linear(c, c)

    def forward(self, hidden_states, scale=1.0):
        return self.b(torch.tanh(self.a(hidden_states))) * scale + hidden_states * 0.1


def _bundle(seed=0):
    teacher = Toy(seed=seed)
    student = copy.deepcopy(teacher)
    teacher.hidden_fn = teacher.hidden

    def install(model, layer, switch):
        model.mix[layer] = switch

    torch.manual_seed(seed + 1)
    return S.Bundle(teacher, student, {1: teacher.mix[1], 2: teacher.mix[2]}, install, lambda layer: Switch(8))


def _batches(seed):
    def get(step):
        g = torch.Generator().manual_seed(1000 * seed + step)
        return torch.randint(0, 17, (8, 12), generator=g)
    return get


def test_stages_chain_and_improve(tmp_path):
    b = _bundle()
    r1 = S.run_stage1(b, _batches(1), S.Stage1Config(steps=150, lr=1e-2), tmp_path / "s1")
    rows = [json.loads(l) for l in open(tmp_path / "s1" / "metrics.jsonl")]
    assert rows[-1]["loss"] < 0.5 * rows[0]["loss"] and r1["layers"] == [1, 2] and (tmp_path / "s1" / "COMPLETE.json").exists()
    eval_ids = _batches(9)(0)
    r2 = S.run_stage2(b, _batches(2), S.Stage2Config(total_tokens=8 * 11 * 60, lr=5e-3), tmp_path / "s2", stage1_dir=tmp_path / "s1",
                      eval_ids=eval_ids)
    assert isinstance(b.student.mix[1], Switch) and isinstance(b.student.mix[0], Mixer)
    assert r2["evaluation_after"]["forward_kl"] < 0.5 * r2["evaluation_before"]["forward_kl"]
    assert json.loads((tmp_path / "s2" / "RUN_CONTRACT.json").read_text())["lineage"]["fingerprint"] == r1["fingerprint"]
    r3 = S.run_stage3(b, lambda step: _batches(3)(step)[:, :4], S.Stage3Config(total_tokens=2500, lr=2e-3, min_gen_tokens=2, max_gen_tokens=8,
                                                                              plateau_steps=4, anchor_kl_weight=0.5),
                      tmp_path / "s3", stage2_dir=tmp_path / "s2", anchor_batches=_batches(4))
    rows = [json.loads(l) for l in open(tmp_path / "s3" / "metrics.jsonl")]
    assert all(r["reverse_kl"] >= 0 and r["anchor_forward_kl"] >= 0 for r in rows) and r3["tokens"] >= 2500
    assert rows[-1]["gen_tokens"] >= rows[0]["gen_tokens"] and r3["gen_tokens"] in (2, 4, 8)


def test_lineage_and_contract_refusals(tmp_path):
    b = _bundle()
    with pytest.raises(ValueError, match="has not finished"):
        S.run_stage2(b, _batches(2), S.Stage2Config(total_tokens=100), tmp_path / "s2", stage1_dir=tmp_path / "nothing")
    S.run_stage1(b, _batches(1), S.Stage1Config(steps=3), tmp_path / "s1")
    with pytest.raises(ValueError, match="expected a stage-2 run"):
        S.run_stage3(b, _batches(3), S.Stage3Config(total_tokens=10), tmp_path / "s3", stage2_dir=tmp_path / "s1")
    with pytest.raises(ValueError, match="different contract"):
        S.run_stage1(_bundle(), _batches(1), S.Stage1Config(steps=4), tmp_path / "s1")
    ckpt = tmp_path / "s1" / json.loads((tmp_path / "s1" / "COMPLETE.json").read_text())["checkpoint"]
    ckpt.write_bytes(ckpt.read_bytes() + b"x")
    with pytest.raises(ValueError, match="differs from its receipt"):
        S.run_stage2(_bundle(), _batches(2), S.Stage2Config(total_tokens=100), tmp_path / "s2b", stage1_dir=tmp_path / "s1")
    with pytest.raises(ValueError):
        S.Stage3Config(min_gen_tokens=4, max_gen_tokens=24)
    with pytest.raises(ValueError, match="anchor"):
        S.Stage3Config(anchor_kl_weight=-1.0)


def test_stage1_resumes_from_its_newest_checkpoint(tmp_path):
    full = S.run_stage1(_bundle(), _batches(1), S.Stage1Config(steps=20, save_every=5), tmp_path / "a")
    # an interrupted copy of the same run: only the step-10 checkpoint and the contract survive
    (tmp_path / "b").mkdir()
    for name in ("RUN_CONTRACT.json", "step-0000010.pt"):
        (tmp_path / "b" / name).write_bytes((tmp_path / "a" / name).read_bytes())
    again = S.run_stage1(_bundle(), _batches(1), S.Stage1Config(steps=20, save_every=5), tmp_path / "b")
    rows = [json.loads(l) for l in open(tmp_path / "b" / "metrics.jsonl")]
    assert [r["step"] for r in rows] == list(range(11, 21))
    assert again["loss"] == pytest.approx(full["loss"], rel=1e-5)
