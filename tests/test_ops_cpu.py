"""CPU numerics tests: delta-rule chunk forms vs recurrences, quantizers, MoE blocks, best-fit packing."""
import itertools
import random

import pytest
import torch

from archlab_b200.data.packing import BestFitPacker, replicated_global_batch
from archlab_b200.models import moe
from archlab_b200.ops import delta_rule as dr
from archlab_b200.ops import quant


def _delta_inputs(B=2, T=150, H=3, K=16, V=24, per_channel=False, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=g)
    k = torch.randn(B, T, H, K, generator=g)
    v = torch.randn(B, T, H, V, generator=g)
    shape = (B, T, H, K) if per_channel else (B, T, H)
    decay = -torch.rand(shape, generator=g) * 0.3
    beta = torch.rand(B, T, H, generator=g)
    return q, k, v, decay, beta


def test_chunk_gated_delta_matches_recurrence():
    q, k, v, decay, beta = _delta_inputs()
    ref = dr.gated_delta_reference(q, k, v, decay, beta)
    for chunk in (16, 64):
        out = dr.chunk_gated_delta_rule(q, k, v, decay, beta, chunk=chunk)
        torch.testing.assert_close(out, ref, atol=2e-5, rtol=1e-4)


def test_chunk_kda_matches_recurrence_and_carries_state():
    q, k, v, g, beta = _delta_inputs(per_channel=True, seed=1)
    ref = dr.kda_recurrent_reference(q, k, v, g, beta)
    out, state = dr.chunk_kda(q, k, v, g, beta, chunk=32, output_final_state=True)
    torch.testing.assert_close(out, ref, atol=2e-5, rtol=1e-4)
    # split the sequence in two and pass the state
    cut = 64
    o1, s1 = dr.chunk_kda(q[:, :cut], k[:, :cut], v[:, :cut], g[:, :cut], beta[:, :cut], chunk=32, output_final_state=True)
    o2, s2 = dr.chunk_kda(q[:, cut:], k[:, cut:], v[:, cut:], g[:, cut:], beta[:, cut:], chunk=32, initial_state=s1,
                          output_final_state=True)
    torch.testing.assert_close(torch.cat([o1, o2], 1), ref, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(s2, state, atol=2e-5, rtol=1e-4)


def test_chunk_kda_backward_matches_recurrence():
    q, k, v, g, beta = _delta_inputs(B=1, T=40, H=2, K=8, V=8, per_channel=True, seed=2)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta)]
    dr.kda_recurrent_reference(*leaves).square().sum().backward()
    want = [t.grad.clone() for t in leaves]
    leaves2 = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta)]
    dr.chunk_kda(*leaves2, chunk=16).square().sum().backward()
    for a, b in zip(leaves2, want):
        torch.testing.assert_close(a.grad, b, atol=1e-4, rtol=1e-3)


def test_causal_conv_is_causal():
    x = torch.randn(2, 12, 6)
    w = torch.randn(6, 4)
    y = dr.causal_conv1d(x, w)
    x2 = x.clone()
    x2[:, 7:] += 1.0
    y2 = dr.causal_conv1d(x2, w)
    torch.testing.assert_close(y[:, :7], y2[:, :7])
    assert not torch.allclose(y[:, 7:], y2[:, 7:])


def test_kda_gate_sign():
    raw = torch.randn(2, 5, 3, 8)
    g = dr.fused_kda_gate(raw, torch.zeros(3), torch.zeros(3, 8))
    assert (g <= 0).all() and g.shape == raw.shape


# ---------------------------------------------------------------------------------- quantizers
def test_pow2_scale_is_exact_ceiling():
    s = torch.tensor([1.0, 1.0000001, 0.75, 3.0, 2.0 ** -20])
    out = quant.pow2_ceil_scale(s)
    assert out.tolist() == [1.0, 2.0, 1.0, 4.0, 2.0 ** -20]


def test_fp8_block_roundtrip_error():
    x = torch.randn(8, 256) * 3
    q, s = quant.fp8_block_quantize(x, 128)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (8, 2)
    back = quant.fp8_block_dequantize(q, s, 128)
    assert ((back - x).abs() <= x.abs() * 2 ** -3 + 1e-3).all()       # e4m3: 3 mantissa bits, pow2 head-room
    assert (torch.log2(s) == torch.log2(s).round()).all()
    wq, ws = quant.fp8_weight_quantize_2d(torch.randn(200, 300), 128)
    assert wq.shape == (200, 300) and ws.shape == (2, 3)
    y = quant.fp8_linear_reference(torch.randn(4, 256), torch.randn(16, 256))
    assert y.shape == (4, 16)


def test_e2m1_rounding_ties_and_stochastic_mean():
    z = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -2.5, 0.2, 5.9])
    got = quant._e2m1_round(z)
    assert got.tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, -2.0, 0.0, 6.0]
    g = torch.Generator().manual_seed(0)
    z = torch.full((20000,), 2.4)
    mean = quant._e2m1_round(z, stochastic=True, generator=g).mean()
    assert abs(mean - 2.4) < 0.02


def test_nvfp4_roundtrip_and_hadamard_cancels():
    x = torch.randn(32, 64)
    vals, bs, ts = quant.nvfp4_quantize(x)
    assert bs.dtype == torch.float8_e4m3fn and bs.shape == (32, 4)
    assert set(vals.abs().unique().tolist()) <= set(quant.E2M1_VALUES)
    back = quant.nvfp4_dequantize(vals, bs, ts)
    assert (back - x).abs().mean() < 0.12 * x.abs().mean() + 0.05
    sign = torch.randint(0, 2, (64,)).float() * 2 - 1
    a, b = torch.randn(8, 64), torch.randn(5, 64)
    ra, rb = quant.random_hadamard_transform(a, sign), quant.random_hadamard_transform(b, sign)
    torch.testing.assert_close(ra @ rb.t(), a @ b.t(), atol=1e-4, rtol=1e-4)


def test_rounded_activation_straight_through():
    x = torch.randn(4, 64, requires_grad=True)
    y = quant.rounded_activation(x, bits=4, block_size=32)
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))
    with pytest.raises(ValueError):
        quant.rounded_activation(x, bits=8, e4m3_scale=True)


def test_stochastic_bf16_unbiased():
    g = torch.Generator().manual_seed(0)
    v = torch.full((50000,), 1.0 + 2 ** -10)
    out = quant.stochastic_bfloat16(v, generator=g).float()
    assert set(out.unique().tolist()) <= {1.0, 1.0 + 2 ** -7}
    assert abs(out.mean() - v[0]) < 2e-4


# ---------------------------------------------------------------------------------- MoE
def test_route_scores_and_bias():
    x, w = torch.randn(10, 8), torch.randn(6, 8)
    for score in ("softmax", "sigmoid", "sqrt_softplus"):
        wt, idx, sc = moe.route(x, w, None, top_k=2, score=score, route_scale=2.5)
        torch.testing.assert_close(wt.sum(-1), torch.full((10,), 2.5))
        assert torch.equal(idx, sc.topk(2).indices)
    bias = torch.zeros(6)
    bias[3] = 100.0
    wt, idx, sc = moe.route(x, w, bias, top_k=2)
    assert (idx == 3).any(-1).all()
    torch.testing.assert_close(wt, sc.gather(1, idx) / sc.gather(1, idx).sum(-1, keepdim=True))   # bias selects only


def test_sparse_moe_matches_dense_loop():
    torch.manual_seed(0)
    m = moe.SparseMoE(16, 24, n_experts=4, top_k=2, n_shared=1, swiglu_limit=7.0)
    m.init_weights(0.3)
    x = torch.randn(3, 5, 16)
    y = m(x)
    x2 = x.reshape(-1, 16)
    w, idx, _ = moe.route(x2, m.router, m.e_score_correction_bias, top_k=2)
    want = m.shared(x2).float()
    for t in range(x2.size(0)):
        for j in range(2):
            e = idx[t, j]
            h = x2[t] @ m.experts.gate_up[e].t()
            a = moe.swiglu_clamped(h[:24], h[24:], 7.0)
            want[t] += w[t, j] * (a @ m.experts.down[e].t())
    torch.testing.assert_close(y.reshape(-1, 16), want, atol=1e-5, rtol=1e-4)
    assert m.last_metrics["load"].sum() == 30
    y.sum().backward()
    assert m.router.grad is not None and m.experts.down.grad.abs().sum() > 0


def test_balance_routers_moves_bias_against_load():
    m = moe.SparseMoE(8, 8, n_experts=4, top_k=1)
    m._cumulative_expert_load = torch.tensor([10.0, 0.0, 5.0, 5.0])
    stats = moe.balance_routers([m], 0.01)
    assert m.e_score_correction_bias.tolist() == pytest.approx([-0.01, 0.01, 0.0, 0.0])
    assert stats["router_dead_fraction_max"] == 0.25 and m._cumulative_expert_load is None
    m._cumulative_expert_load = torch.tensor([10.0, 0.0, 5.0, 5.0])
    before = m.e_score_correction_bias.clone()
    moe.balance_routers([m], 0.01, proportional=True)
    delta = m.e_score_correction_bias - before
    assert abs(float(delta.sum())) < 1e-7 and delta[1] > 0 > delta[0]


# ---------------------------------------------------------------------------------- packing
def _docs(seed=0):
    rng = random.Random(seed)
    while True:
        yield [rng.randrange(1, 100) for _ in range(rng.randrange(1, 40))]


def test_best_fit_rows_start_with_bos_and_replay():
    p = BestFitPacker(_docs(), batch_size=4, seq_len=32, buffer_size=50, bos_token=0)
    batches = [p.next_batch() for _ in range(3)]
    for x, y, st in batches:
        assert x.shape == (4, 32) and (x[:, 0] == 0).all()
        assert torch.equal(x[:, 1:], y[:, :-1])
    q = BestFitPacker(_docs(), batch_size=4, seq_len=32, buffer_size=50, bos_token=0)
    q.seek(2)
    x, y, st = q.next_batch()
    assert st["batch_index"] == 2 and torch.equal(x, batches[2][0])


def test_replicated_global_batch_pads_with_ignored_targets():
    parts = []
    for r in range(3):
        p = BestFitPacker(_docs(1), batch_size=4, seq_len=16, buffer_size=20, bos_token=0)
        parts.append(replicated_global_batch(p, r, 3))
    ys = torch.cat([y for _, y, _ in parts])
    assert ys.shape[0] == 6 and (ys[4:] == -1).all() and (ys[:4] >= 0).all()


def test_chunk_forms_survive_strong_decay():
    q, k, v, g, beta = _delta_inputs(B=1, T=130, H=2, K=8, V=8, per_channel=True, seed=3)
    g = g * 80.0                                    # cumulative log-decay far below exp() underflow
    ref = dr.kda_recurrent_reference(q, k, v, g, beta)
    out = dr.chunk_kda(q, k, v, g, beta)
    assert torch.isfinite(out).all()
    torch.testing.assert_close(out, ref, atol=2e-5, rtol=1e-4)
