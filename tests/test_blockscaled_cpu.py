"""Block-scaled operand format: the PyTorch statement of the quantisers, the chunked scale layout and the GEMM."""
import torch

from archlab_b200.ops import blockscaled as bs


def test_scale_chunk_layout_is_a_bijection():
    idx = bs.sf_index(300, 12, 3)
    flat = idx.view(-1)
    assert flat.unique().numel() == flat.numel() and int(flat.max()) < bs.sf_bytes("fp8", 300, 12 * 32)
    # row 37 of tile 0, scale 5 -> chunk 1, lane 5, quarter 1, byte 1
    assert int(idx[37, 5]) == 1 * 512 + 5 * 16 + 1 * 4 + 1
    assert int(idx[128, 0]) == 3 * 512


def test_fp8_rules_decode_close_to_the_source():
    torch.manual_seed(0)
    x = torch.randn(200, 320) * torch.logspace(-2, 2, 320)
    xb = x.bfloat16().float()
    for block in (32, 128, -128):
        d = bs.decode(bs.quantize_fp8_reference(x.bfloat16(), block))
        # e4m3 keeps 3 mantissa bits: 2^-4 of the element for normal values, of the block maximum / 2^8 below that
        assert (d - xb).norm() / xb.norm() < 0.04, block
        if block == 32:
            bmax = xb.view(200, 10, 32).abs().amax(-1).repeat_interleave(32, 1)
            assert ((d - xb).abs() <= xb.abs() * 2 ** -4 + bmax * 2 ** -9).all()
    # 1 x 128: one exponent per row and 128 columns, repeated over the four sub-blocks
    op = bs.quantize_fp8_reference(x.bfloat16(), 128)
    e = op.sf[bs.sf_index(200, 12, op.chunks_k)]
    assert torch.equal(e[:, 0], e[:, 3]) and torch.equal(e[:, 4], e[:, 7])
    # 128 x 128: one exponent per block of rows too
    op = bs.quantize_fp8_reference(x.bfloat16(), -128)
    e = op.sf[bs.sf_index(200, 12, op.chunks_k)]
    assert (e[:128, 0] == e[0, 0]).all() and (e[128:, 0] == e[128, 0]).all()


def test_fp8_scales_are_the_smallest_powers_of_two_that_fit():
    x = torch.tensor([[448.0] * 32 + [480.0] * 32 + [0.0] * 32 + [2.0 ** -10] * 32]).bfloat16()
    op = bs.quantize_fp8_reference(x, 32)
    e = op.sf[bs.sf_index(1, 4, 1)].view(-1).int() - 127
    assert e.tolist() == [0, 1, -22, -18]      # the all-zero block sits at the 1e-4 floor
    assert torch.allclose(bs.decode(op), x.float())


def test_nvfp4_round_trip_and_hadamard_cancels_in_the_product():
    torch.manual_seed(1)
    a, b = torch.randn(64, 256).bfloat16(), torch.randn(48, 256).bfloat16()
    exact = a.float() @ b.float().t()
    plain = bs.reference_gemm(bs.quantize_nvfp4_reference(a), bs.quantize_nvfp4_reference(b, two_d=True))
    rht = bs.reference_gemm(bs.quantize_nvfp4_reference(a, hadamard_seed=7), bs.quantize_nvfp4_reference(b, hadamard_seed=7))
    for got in (plain, rht):
        assert (got - exact).norm() / exact.norm() < 0.15
    h = bs.hadamard16(7)
    assert torch.allclose(h @ h.t(), torch.eye(16), atol=1e-6)
    # decode is exact for values on the grid with unit scales
    grid = torch.tensor([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0, 0.0]])
    op = bs.quantize_nvfp4_reference(grid.bfloat16(), amax=torch.tensor(bs.NVFP4_RANGE / 1.0 * 6.0 / 6.0))
    assert torch.allclose(bs.decode(op), grid, atol=0.0)


def test_nvfp4_stochastic_rounding_is_unbiased():
    x = torch.full((256, 16), 1.3).bfloat16()
    x[:, 0] = 6.0                                   # pins the block scale
    u = torch.rand(256, 16, generator=torch.Generator().manual_seed(3))
    op = bs.quantize_nvfp4_reference(x, uniforms=u)
    d = bs.decode(op)[:, 1:]
    assert {round(v, 4) for v in d.unique().tolist()} <= {1.0, 1.5} and abs(float(d.mean()) - float(x[0, 1])) < 0.03


def test_cpu_gemm_and_grouped_form():
    torch.manual_seed(2)
    a = torch.randn(512, 128).bfloat16()
    w = torch.randn(3 * 128, 128).bfloat16()
    qa, qw = bs.quantize_fp8(a, 128), bs.quantize_fp8(w, -128)
    got = bs.grouped_gemm(qa, qw, torch.tensor([2, 0], dtype=torch.int32), 3, 128).float()
    exact = torch.cat([a[:256].float() @ w[256:384].float().t(), a[256:].float() @ w[:128].float().t()])
    assert (got - exact).norm() / exact.norm() < 0.06
    full = bs.gemm(qa, qw, out_dtype=torch.float32)
    assert (full - a.float() @ w.float().t()).norm() / (a.float() @ w.float().t()).norm() < 0.06
