"""NativeLinear on the tcgen05 GEMM kernels against fp32 matmul: forward, data gradient, weight gradient."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("rows,k,n", [(300, 256, 512), (2048, 1280, 5120), (77, 128, 136)])
def test_three_gemms_match_fp32(rows, k, n):
    from archlab_b200.ops.native_linear import native_linear

    torch.manual_seed(0)
    x = (torch.randn(3, rows, k, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    dy = (torch.randn(3, rows, n, device="cuda") * 0.5).bfloat16()
    y = native_linear(x, w)
    y.backward(dy)
    xf, wf, df = x.detach().float(), w.detach().float(), dy.float()
    assert _rel(y, xf @ wf.t()) < 1e-2
    assert _rel(x.grad, df @ wf) < 1e-2
    assert _rel(w.grad, df.flatten(0, 1).t() @ xf.flatten(0, 1)) < 1e-2
