"""FP8 pair-CTA GEMM (kind::f8f6f4) against the fp32 product of the same 8-bit operands; Float8Linear gradients."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,adt,bdt", [(512, 768, 1024, "e4m3", "e4m3"), (300, 260, 208, "e5m2", "e4m3"), (256, 256, 4096, "e5m2", "e5m2")])
def test_fp8_gemm_matches_fp32_product(M, N, K, adt, bdt):
    from archlab_b200.ops import fp8, native

    torch.manual_seed(0)
    dt = {"e4m3": fp8.E4M3, "e5m2": fp8.E5M2}
    a = (torch.randn(M, K, device="cuda") * 2).to(dt[adt])
    b = (torch.randn(N, K, device="cuda") * 2).to(dt[bdt])
    out = fp8.fp8_gemm(a, b, 0.5, torch.float32)
    torch.cuda.synchronize()
    native.check_status()
    ref = 0.5 * (a.float() @ b.float().t())
    assert (out - ref).norm() / ref.norm() < 1e-3


def test_float8_linear_training_step():
    from archlab_b200.ops import fp8

    torch.manual_seed(0)
    lin = fp8.Float8Linear(1024, 768, bias=False).cuda().bfloat16()
    x = torch.randn(512, 1024, device="cuda").bfloat16().requires_grad_(True)
    g = torch.randn(512, 768, device="cuda").bfloat16()
    y = lin(x)
    y.backward(g)
    yr = x.detach().float() @ lin.weight.float().t()
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
    assert rel(y, yr) < 0.06
    assert rel(x.grad, g.float() @ lin.weight.float()) < 0.12 and rel(lin.weight.grad, g.float().t() @ x.detach().float()) < 0.12
