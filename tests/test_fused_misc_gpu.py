"""Single-pass model-zoo kernels against their PyTorch statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def test_rmsnorm_variants():
    from archlab_b200.models.blocks import rms_norm
    from archlab_b200.ops import fused_misc as fm

    x = torch.randn(300, 4 * 256, device="cuda").bfloat16()
    w = torch.randn(4 * 256, device="cuda") * 0.1
    for groups, zc in ((1, False), (4, True), (4, False)):
        width = x.size(-1) // groups
        got = fm.rmsnorm(x, w, groups=groups, zero_centered=zc)
        xf = x.float().unflatten(-1, (groups, width))                      # plain fp32 statement of the op
        gain = (1.0 + w.view(groups, width)) if zc else w.view(groups, width)
        want = (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + 1e-6) * gain).flatten(-2)
        assert _rel(got, want) < 6e-3
        # the model-level function routes [.., groups, width] inputs with a [groups, width] gain to the same kernel
        via = rms_norm(x.unflatten(-1, (groups, width)), w.view(groups, width), zero_centered=zc).flatten(-2)
        assert _rel(via, want) < 6e-3
    xf = x.float()
    assert _rel(fm.rmsnorm(x), xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + 1e-6)) < 6e-3
    assert _rel(rms_norm(x), xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + 1e-6)) < 6e-3


def test_rope_styles():
    from archlab_b200.models.blocks import apply_rope, rope_tables
    from archlab_b200.ops import fused_misc as fm

    x = torch.randn(2, 33, 3, 64, device="cuda").bfloat16()
    cos, sin = rope_tables(33, 32, device="cuda")
    for inter in (False, True):
        want = apply_rope(x.float(), cos, sin, style="interleaved" if inter else "half", rot_dim=32)   # fp32 PyTorch path
        got = fm.rope_(x.clone(), cos, sin, rot_dim=32, interleaved=inter)
        assert _rel(got, want) < 6e-3 and torch.equal(got[..., 32:], x[..., 32:])


def test_router_topk_matches_statement():
    from archlab_b200.models.moe import route
    from archlab_b200.ops import fused_misc as fm

    torch.manual_seed(0)
    x = torch.randn(77, 256, device="cuda").bfloat16()
    w = (torch.randn(64, 256, device="cuda") * 0.2).bfloat16()
    bias = torch.randn(64, device="cuda") * 0.05
    for score in ("softmax", "sigmoid", "sqrt_softplus"):
        gw, gi, gs = fm.router_topk(x, w, bias, top_k=6, score=score, route_scale=1.5, return_scores=True)
        ww, wi, ws = route(x, w, bias, top_k=6, score=score, route_scale=1.5)
        assert _rel(gs, ws) < 2e-3
        same = (gi.sort(-1).values == wi.sort(-1).values).all(-1).float().mean()
        assert same > 0.97                                  # near-ties may order differently in fp32
        torch.testing.assert_close(gw.sum(-1), torch.full((77,), 1.5, device="cuda"), atol=1e-3, rtol=1e-3)


def test_causal_conv_and_hash():
    from archlab_b200.models.blocks import NgramHash
    from archlab_b200.ops import delta_rule, fused_misc as fm

    x = torch.randn(2, 50, 48, device="cuda").bfloat16()
    w = torch.randn(48, 4, device="cuda") * 0.3
    for dil in (1, 3):
        assert _rel(fm.causal_conv1d(x, w, dilation=dil), delta_rule.causal_conv1d(x.float(), w, dilation=dil)) < 8e-3
    h = NgramHash(1000, 3, 2, [101, 103, 107, 109], eos=0).cuda()
    t = torch.randint(0, 1000, (3, 40), device="cuda")
    t[:, 7] = 0
    got = fm.ngram_hash(t, h.multipliers, h.sizes, h.offsets, ngram=3, heads_per_order=2, eos=0)
    assert torch.equal(got, h(t))


def test_quantizers():
    from archlab_b200.ops import fused_misc as fm, quant

    x = (torch.randn(64, 512, device="cuda") * 3).bfloat16()
    q, s = fm.fp8_block_quantize(x)
    rq, rs = quant.fp8_block_quantize(x)
    assert torch.equal(s, rs) and _rel(q.float(), rq.float()) < 1e-3
    vals, bs, ts = fm.nvfp4_quantize(x)
    rv, rb, _ = quant.nvfp4_quantize(x, tensor_scale=ts)
    assert torch.equal(bs.float(), rb.float())
    assert (vals.float() == rv).float().mean() > 0.995       # bf16 input division rounding at grid ties
    f = torch.full((100000,), 1.0 + 2 ** -10, device="cuda")
    out = fm.stochastic_bf16(f, seed=3).float()
    assert set(out.unique().tolist()) <= {1.0, 1.0 + 2 ** -7} and abs(float(out.mean()) - float(f[0])) < 2e-4
