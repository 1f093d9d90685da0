"""Block-scaled tcgen05 GEMMs (kind::mxf8f6f4 / kind::mxf4nvf4) and their quantisers against the PyTorch statement
of the same format: quantiser bytes, then the GEMM against the fp32 product of the decoded operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


@pytest.mark.parametrize("block", [32, 128, -128])
@pytest.mark.parametrize("rows,K,e5m2", [(256, 512, False), (300, 1184, False), (128, 256, True)])
def test_fp8_quantiser_matches_the_reference_bytes(block, rows, K, e5m2):
    from archlab_b200.ops import blockscaled as bs

    torch.manual_seed(0)
    x = (torch.randn(rows, K, device="cuda") * torch.logspace(-3, 3, K, device="cuda")).bfloat16()
    got = bs.quantize_fp8(x, block, e5m2)
    ref = bs.quantize_fp8_reference(x, block, e5m2)
    assert torch.equal(got.data, ref.data)
    n_sf = -(-K // 32)
    idx = bs.sf_index(rows, n_sf, ref.chunks_k, "cuda")
    assert torch.equal(got.sf[idx], ref.sf[idx])


@pytest.mark.parametrize("two_d,seed", [(False, 0), (True, 0), (False, 11)])
def test_nvfp4_quantiser_matches_the_reference_bytes(two_d, seed):
    from archlab_b200.ops import blockscaled as bs

    torch.manual_seed(1)
    rows, K = 272, 832
    x = (torch.randn(rows, K, device="cuda") * 3).bfloat16()
    got = bs.quantize_nvfp4(x, two_d=two_d, hadamard_seed=seed)
    ref = bs.quantize_nvfp4_reference(x, two_d=two_d, hadamard_seed=seed)
    idx = bs.sf_index(rows, K // 16, ref.chunks_k, "cuda")
    if seed == 0:
        assert torch.equal(got.sf[idx], ref.sf[idx])
        assert int((got.data != ref.data).sum()) == 0, f"{int((got.data != ref.data).sum())} of {ref.data.numel()} bytes differ"
    else:       # the transform's sums round differently in the two orders of addition: compare decoded values
        assert _rel(bs.decode(got), bs.decode(ref)) < 0.02


def test_nvfp4_stochastic_rounding_on_the_device_is_unbiased():
    from archlab_b200.ops import blockscaled as bs

    x = torch.full((2048, 64), 1.3, device="cuda").bfloat16()
    x[:, ::16] = 6.0
    a = bs.decode(bs.quantize_nvfp4(x, sr_seed=5))
    b = bs.decode(bs.quantize_nvfp4(x, sr_seed=6))
    body = a[:, 1:16]
    assert {round(v, 3) for v in body.unique().tolist()} <= {1.0, 1.5}
    assert abs(float(body.mean()) - float(x[0, 1])) < 0.01 and not torch.equal(a, b)


@pytest.mark.parametrize("M,N,K,ablock,bblock", [(256, 256, 128, 32, 32), (512, 768, 1024, 128, -128), (300, 260, 416, 32, 32),
                                                 (1024, 1408, 2048, 128, -128)])
def test_mxfp8_gemm_matches_the_decoded_product(M, N, K, ablock, bblock):
    from archlab_b200.ops import blockscaled as bs, native

    torch.manual_seed(2)
    a = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 2, K, device="cuda")).bfloat16()
    b = (torch.randn(N, K, device="cuda") * torch.logspace(2, -2, K, device="cuda")).bfloat16()
    qa, qb = bs.quantize_fp8(a, ablock), bs.quantize_fp8(b, bblock)
    out = bs.gemm(qa, qb, alpha=0.5, out_dtype=torch.float32)
    torch.cuda.synchronize()
    native.check_status()
    ref = bs.reference_gemm(qa, qb, 0.5)
    assert _rel(out, ref) < 1e-3
    assert _rel(bs.gemm(qa, qb, alpha=0.5), ref) < 5e-3                       # bf16 output through TMA stores
    assert _rel(out, 0.5 * a.float() @ b.float().t()) < 0.06                  # and the format itself is close


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (512, 384, 1024), (300, 520, 832)])
def test_nvfp4_gemm_matches_the_decoded_product(M, N, K):
    from archlab_b200.ops import blockscaled as bs, native

    torch.manual_seed(3)
    a = (torch.randn(M, K, device="cuda") * 2).bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    qa, qb = bs.quantize_nvfp4(a), bs.quantize_nvfp4(b, two_d=(N % 16 == 0))
    out = bs.gemm(qa, qb, out_dtype=torch.float32)
    torch.cuda.synchronize()
    native.check_status()
    ref = bs.reference_gemm(qa, qb)
    assert _rel(out, ref) < 1e-3
    assert _rel(out, a.float() @ b.float().t()) < 0.2
    ha, hb = bs.quantize_nvfp4(a, hadamard_seed=9, sr_seed=3), bs.quantize_nvfp4(b, hadamard_seed=9)
    assert _rel(bs.gemm(ha, hb, out_dtype=torch.float32), a.float() @ b.float().t()) < 0.25


@pytest.mark.parametrize("kind", ["fp8", "nvfp4"])
def test_grouped_block_scaled_gemm(kind):
    from archlab_b200.ops import blockscaled as bs, native

    torch.manual_seed(4)
    G, Nw, K = 3, 384, 512
    a = torch.randn(4 * 256, K, device="cuda").bfloat16()
    w = torch.randn(G * Nw, K, device="cuda").bfloat16()
    groups = torch.tensor([2, 0, 0, 1], dtype=torch.int32, device="cuda")
    if kind == "fp8":
        qa, qw = bs.quantize_fp8(a, 128), bs.quantize_fp8(w, -128)
    else:
        qa, qw = bs.quantize_nvfp4(a), bs.quantize_nvfp4(w, two_d=True)
    out = bs.grouped_gemm(qa, qw, groups, G, Nw)
    torch.cuda.synchronize()
    native.check_status()
    da, dw = bs.decode(qa), bs.decode(qw).view(G, Nw, K)
    ref = torch.cat([da[t * 256:(t + 1) * 256] @ dw[g].t() for t, g in enumerate(groups.tolist())])
    assert _rel(out, ref) < 5e-3


def test_block_fp8_linear_forward_and_straight_through_backward():
    from archlab_b200.ops import blockscaled as bs, native

    torch.manual_seed(5)
    x = torch.randn(4, 96, 1024, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(768, 1024, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    g = torch.randn(4, 96, 768, device="cuda").bfloat16()
    y = bs.block_fp8_linear(x, w)
    y.backward(g)
    torch.cuda.synchronize()
    native.check_status()
    xf, wf = x.detach().float(), w.detach().float()
    assert _rel(y, xf @ wf.t()) < 0.05
    # the gradients ignore the rounding: they are the bf16 products against the unrounded operands
    assert _rel(x.grad, g.float() @ wf) < 0.01
    assert _rel(w.grad, g.float().reshape(-1, 768).t() @ xf.reshape(-1, 1024)) < 0.01


def test_grouped_linear_fp8_forward_matches_bf16_path():
    from archlab_b200.ops import grouped, native

    torch.manual_seed(6)
    E, N, K = 3, 256, 512
    seg, seg_pad = [200, 0, 300], [256, 0, 512]
    x = torch.randn(sum(seg_pad), K, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(E, N, K, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    tiles = grouped.tile_groups(seg_pad, "cuda")
    y8 = grouped.grouped_linear(x, w, tiles, seg, seg_pad, fp8=True)
    y16 = grouped.grouped_linear(x, w, tiles, seg, seg_pad)
    torch.cuda.synchronize()
    native.check_status()
    live = torch.cat([torch.arange(0, 200), torch.arange(256, 556)]).cuda()
    assert _rel(y8[live], y16[live]) < 0.05
    y8[live].float().square().sum().backward()
    assert torch.isfinite(x.grad[live]).all() and torch.isfinite(w.grad).all()


def test_nvfp4_linear_three_products_on_the_fp4_path():
    from archlab_b200.ops import blockscaled as bs, native

    torch.manual_seed(7)
    x = torch.randn(512, 1024, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(768, 1024, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    g = torch.randn(512, 768, device="cuda").bfloat16()
    assert bs.nvfp4_supported(x, w)
    y = bs.nvfp4_linear(x, w, seed=3)
    y.backward(g)
    torch.cuda.synchronize()
    native.check_status()
    xf, wf, gf = x.detach().float(), w.detach().float(), g.float()
    assert _rel(y, xf @ wf.t()) < 0.2
    assert _rel(x.grad, gf @ wf) < 0.25
    assert _rel(w.grad, gf.t() @ xf) < 0.25
    # stochastic rounding: another seed gives other gradients with the same expectation
    x2 = x.detach().clone().requires_grad_(True)
    bs.nvfp4_linear(x2, w.detach(), seed=5).backward(g)
    assert not torch.equal(x2.grad, x.grad) and _rel(x2.grad, gf @ wf) < 0.25


def test_converted_model_trains_a_few_steps_in_nvfp4():
    from archlab_b200.ops import blockscaled as bs

    torch.manual_seed(8)
    # fp32 master weights (the layers cast to bf16 and quantise per call), bf16 activations
    net = torch.nn.Sequential(torch.nn.Linear(256, 512, bias=False), torch.nn.GELU(), torch.nn.Linear(512, 256, bias=False)).cuda()
    rep = bs.convert_linears(net, "nvfp4")
    assert len(rep["converted"]) == 2
    opt = torch.optim.Adam(net.parameters(), lr=3e-3)
    x = torch.randn(256, 256, device="cuda").bfloat16()
    target = (x.float() @ torch.randn(256, 256, device="cuda") * 0.05).tanh()
    losses = []
    for step in range(60):
        bs.set_step(net, step)
        loss = (net(x).float() - target).square().mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.7 * losses[0], losses[::10]
