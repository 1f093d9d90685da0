"""tcgen05 GEMM against the fp32 PyTorch statement of the same arithmetic."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, a_mn, b_mn, batch=0, epi=0, out_dtype=torch.bfloat16, alpha=1.0, beta=0.0):
    from archlab_b200.ops import gemm as G, native

    dev = "cuda"
    sh = (lambda r, c: (batch, r, c)) if batch else (lambda r, c: (r, c))
    a = torch.randn(sh(K, M) if a_mn else sh(M, K), device=dev).bfloat16()
    b = torch.randn(sh(K, N) if b_mn else sh(N, K), device=dev).bfloat16()
    aux = None
    if epi in (G.EPI_AXPBY, G.EPI_MUL_DRELU2):
        aux = torch.randn(sh(M, N), device=dev).abs().to(out_dtype if epi == G.EPI_AXPBY else torch.bfloat16)
    ref = G.gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, aux=aux, epi=epi, alpha=alpha, beta=beta,
                           out_dtype=torch.float32)
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, aux=aux, epi=epi, alpha=alpha, beta=beta, out_dtype=out_dtype)
    torch.cuda.synchronize()
    native.check_status()
    rel = ((out.float() - ref).norm() / ref.norm()).item()
    assert rel < (1e-5 if out_dtype == torch.float32 else 4e-3), rel


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 512, 256), (200, 328, 136), (1024, 1280, 512)])
def test_orientations(shape, a_mn, b_mn):
    torch.manual_seed(0)
    _case(*shape, a_mn, b_mn)


def test_fp32_output_and_accumulate():
    torch.manual_seed(1)
    _case(512, 1024, 2048, 1, 1, out_dtype=torch.float32)
    _case(512, 1024, 256, 1, 1, epi=1, out_dtype=torch.float32, alpha=1.0, beta=1.0)


def test_batched_and_epilogues():
    torch.manual_seed(2)
    _case(640, 640, 640, 0, 0, batch=5)
    _case(640, 640, 640, 0, 1, batch=5, epi=1, alpha=0.5, beta=2.0)
    _case(512, 1024, 256, 0, 0, epi=2)
    _case(512, 1024, 256, 0, 1, epi=3)
