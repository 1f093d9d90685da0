"""Headwise Muon, Muown, sharded Adafactor, Sinkhorn tables, recipes."""
import math

import pytest
import torch

from archlab_b200.optim import extra as ox
from archlab_b200.optim.recipes import OPTIMIZATION_RECIPES, get_optimization_recipe


def test_orthogonalized_direction_has_unit_singular_values():
    torch.manual_seed(0)
    g = torch.randn(3, 8, 20)
    u = ox.orthogonalized_direction(g)
    s = torch.linalg.svdvals(u)
    assert (s > 0.6).all() and (s < 1.3).all()
    assert torch.equal(ox.orthogonalized_direction(torch.zeros(4, 6)), torch.zeros(4, 6))
    tall = ox.orthogonalized_direction(torch.randn(20, 8))
    assert tall.shape == (20, 8)


def test_headwise_muon_updates_heads_independently():
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(8, 6))
    opt = ox.HeadwiseMuon([{"params": [p], "head_dim": 4}], lr=0.1, weight_decay=0.0)
    before = p.detach().clone()
    p.grad = torch.cat([torch.randn(4, 6), torch.zeros(4, 6)])
    opt.step()
    assert not torch.equal(p[:4], before[:4]) and torch.equal(p[4:], before[4:])      # zero-gradient head untouched
    rms = (p[:4] - before[:4]).square().mean().sqrt()
    assert 0.005 < float(rms.detach()) < 0.05                                          # ~ lr * update_rms * O(1)
    with pytest.raises(ValueError):
        ox.HeadwiseMuon([{"params": [torch.nn.Parameter(torch.randn(7, 3))], "head_dim": 4}])


def test_muown_keeps_weight_normalised_form_and_descends():
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(6, 10))
    target = torch.randn(6, 10)
    opt = ox.Muown([w], lr=0.05)
    losses = []
    for _ in range(30):
        loss = (w - target).square().mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0]
    st = opt.state[w]
    torch.testing.assert_close(w.detach().norm(dim=1, keepdim=True), st["g"].abs(), atol=1e-5, rtol=1e-5)
    w16 = torch.nn.Parameter(torch.randn(4, 4))
    o16 = ox.Muown([w16], momentum_dtype=torch.float16)
    w16.grad = torch.randn(4, 4) * 1e-6
    o16.step()
    assert o16.state[w16]["momentum_buffer"].dtype == torch.float16 and float(o16.state[w16]["momentum_scale"]) < 1


def test_adafactor_descends_and_rounds_stochastically():
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(3, 16, 8))
    b = torch.nn.Parameter(torch.randn(8))
    target = torch.zeros(3, 16, 8)
    opt = ox.ShardedAdafactor([w, b], lr=0.05, chunk_elements=40)
    first = None
    for _ in range(40):
        loss = (w - target).square().mean() + b.square().mean()
        first = first if first is not None else float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < first and opt.last_metrics["updated_parameter_tensors"] == 2
    assert opt.state[w]["row"].shape == (3, 16, 1) and opt.state[w]["col"].shape == (3, 1, 8)
    wb = torch.nn.Parameter(torch.ones(4, 4, dtype=torch.bfloat16))
    ob = ox.ShardedAdafactor([wb], lr=1e-3)
    wb.grad = torch.ones(4, 4, dtype=torch.bfloat16)
    ob.step()
    assert wb.dtype == torch.bfloat16 and set(wb.detach().float().unique().tolist()) <= {1.0, 1.0 - 2 ** -8, 1.0 - 2 ** -7}


def test_sinkhorn_direction_normalises_rows_and_columns():
    torch.manual_seed(0)
    u = torch.randn(12, 5) * torch.logspace(-1, 1, 12)[:, None]
    d = ox.sinkhorn_direction(u)
    torch.testing.assert_close(d.norm(dim=1), torch.full((12,), math.sqrt(5.0)), atol=0.35, rtol=0.2)
    assert torch.equal(ox.sinkhorn_direction(torch.zeros(3, 4)), torch.zeros(3, 4))
    u2 = u.clone()
    u2[0] = 1e-9
    assert torch.equal(ox.sinkhorn_direction(u2)[0], torch.zeros(5))                   # below the row threshold
    with pytest.raises(ValueError):
        ox.sinkhorn_direction(u, steps=4)
    t = torch.nn.Parameter(torch.randn(12, 5))
    opt = ox.SinkhornTables([t], lr=0.1)
    before = t.detach().clone()
    t.grad = torch.randn(12, 5)
    opt.step()
    assert not torch.equal(t, before) and opt.state[t]["step"] == 1


def test_recipes_are_single_hypotheses():
    assert len(OPTIMIZATION_RECIPES) == 39 and "baseline" in OPTIMIZATION_RECIPES
    r = get_optimization_recipe("muonh-tuned-aux")
    assert (r.matrix_optimizer, r.matrix_lr, r.scalar_lr) == ("muonh", 0.018, 0.0195)
    assert get_optimization_recipe("z-loss-5e-6-clip01").gradient_clip == 0.1
    assert get_optimization_recipe("adam-every-2").adam_update_every == 2
    with pytest.raises(ValueError):
        get_optimization_recipe("nope")
