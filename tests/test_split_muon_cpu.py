"""Layer-wise distributed Muon with logical row splits: the orthogonalisation against a literal statement of the
eight-step schedule, the split rule, placement, and a two-rank run against the single-process update."""
import math
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from archlab_b200.optim.split_muon import (POLAR_EXPRESS_8, SplitRowsMuon, logical_matrices, lpt_placement, muon_recipe,
                                           orthogonalize)
from conftest import join_ranks


def _literal(m):
    t = m.size(-2) > m.size(-1)
    v = m.mT if t else m
    v = v / v.square().sum(dim=(-2, -1), keepdim=True).sqrt().clamp_min(1e-14)
    for a, b, c in POLAR_EXPRESS_8:
        g = v @ v.mT
        v = a * v + (b * g + c * (g @ g)) @ v
    return v.mT if t else v


@pytest.mark.parametrize("shape", [(3, 16, 48), (2, 40, 24), (1, 32, 32)])
def test_orthogonalize_matches_the_schedule_and_is_near_orthogonal(shape):
    torch.manual_seed(0)
    m = torch.randn(shape)
    got = orthogonalize(m, bf16=False)
    torch.testing.assert_close(got, _literal(m), rtol=1e-4, atol=1e-5)
    small = got if shape[1] <= shape[2] else got.mT
    gram = small @ small.mT
    assert (gram - torch.eye(gram.size(-1))).abs().max() < 0.35     # singular values pushed towards one


def test_logical_split_rule_and_placement():
    w = torch.arange(24.0).view(6, 4)
    assert logical_matrices(w, 2).shape == (3, 2, 4) and logical_matrices(w, None).shape == (1, 6, 4)
    assert logical_matrices(torch.zeros(5, 8, 3), 4).shape == (10, 4, 3)       # stacked experts: E x R / r matrices
    with pytest.raises(ValueError):
        logical_matrices(w, 4)
    assert lpt_placement([5, 9, 2, 7, 1], 2) == [1, 0, 0, 1, 0]                 # 9+2+1 | 7+5: both ranks carry 12
    assert muon_recipe()["newton_schulz_steps"] == 8


def _model(seed=0):
    torch.manual_seed(seed)
    m = torch.nn.ModuleDict({"q": torch.nn.Linear(24, 32, bias=False), "up": torch.nn.Linear(24, 40, bias=False),
                             "norm": torch.nn.LayerNorm(24)})
    for lin, rows in ((m["q"], 8), (m["up"], None)):
        lin.weight.archlab_optimizer = "muon"
        if rows:
            lin.weight.archlab_muon_split_rows = rows
    return m


def _loss(m, x):
    h = m["norm"](x)
    return (m["q"](h).square().mean() + m["up"](h).tanh().mean())


def test_update_rule_on_one_rank():
    m = _model()
    opt = SplitRowsMuon(m.named_parameters(), lr=0.05, weight_decay=0.1, bf16=False)
    assert set(opt.placement()) == {"q.weight", "up.weight"}
    w0 = m["q"].weight.detach().clone()
    _loss(m, torch.randn(16, 24)).backward()
    g = m["q"].weight.grad.clone()
    opt.step()
    direction = g + 0.95 * g                                  # first step: momentum buffer = g, Nesterov look-ahead
    upd = orthogonalize(direction.view(4, 8, 24), bf16=False) * (0.2 * math.sqrt(24))
    torch.testing.assert_close(m["q"].weight.detach(), w0 * (1 - 0.05 * 0.1) - 0.05 * upd.view(32, 24), rtol=1e-5, atol=1e-6)
    assert m["q"].weight.grad is None and m["norm"].weight.grad is not None     # untagged parameters are left alone


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m, ref = _model(), _model()
    opt = SplitRowsMuon(m.named_parameters(), lr=0.05, bf16=False)
    solo = SplitRowsMuon(ref.named_parameters(), lr=0.05, bf16=False, group=dist.new_group([rank]))
    g = torch.Generator().manual_seed(5)
    data = torch.randn(2, 8, 24, generator=g)
    for _ in range(3):
        _loss(m, data[rank]).backward()
        opt.reduce_gradients()
        opt.step()
        (0.5 * (_loss(ref, data[0]) + _loss(ref, data[1]))).backward()        # the mean over both ranks' batches
        solo.step()
    ok = all(torch.allclose(a, b, atol=1e-5) for a, b in zip(m.parameters(), ref.parameters()))
    owned = sum(e.momentum is not None for e in opt.entries)
    q.put((rank, ok, owned, sorted(opt.placement().values())))
    dist.destroy_process_group()


def test_two_ranks_follow_the_single_process_run():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29673, q)) for r in range(2)]
    for p in procs:
        p.start()
    join_ranks(procs, 180)
    out = sorted(q.get(timeout=5) for _ in range(2))
    assert all(ok for _, ok, _, _ in out)
    assert [owned for _, _, owned, _ in out] == [1, 1] and out[0][3] == [0, 1]     # each rank keeps state for one matrix


def test_qwen38_tags_survive_meta_materialisation_and_give_per_head_matrices():
    from archlab_b200.models.factory import build_model

    model = build_model("qwen38_tiny", {"sequence_len": 16})
    tagged = {n: p for n, p in model.named_parameters() if getattr(p, "archlab_optimizer", None) == "muon"}
    assert tagged, "factory-built models keep their optimizer tags"
    split = {n: p.archlab_muon_split_rows for n, p in tagged.items() if hasattr(p, "archlab_muon_split_rows")}
    assert any(n.endswith("qkv.weight") for n in split) or any(n.endswith("q_gate.weight") for n in split)
    for n, rows in split.items():
        assert logical_matrices(tagged[n], rows).shape[-2] == rows and tagged[n].shape[-2] % rows == 0
    opt = SplitRowsMuon(model.named_parameters(), bf16=False)
    assert set(opt.placement()) == set(tagged)
