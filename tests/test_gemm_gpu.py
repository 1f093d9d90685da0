"""tcgen05 GEMM against the fp32 PyTorch statement of the same arithmetic."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, a_mn, b_mn, batch=0, epi=0, out_dtype=torch.bfloat16, alpha=1.0, beta=0.0, impl=None):
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
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, aux=aux, epi=epi, alpha=alpha, beta=beta, out_dtype=out_dtype,
                 impl=impl)
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


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 256), (304, 328, 136), (2048, 1280, 512)])
def test_pair_kernel_orientations(shape, a_mn, b_mn):
    """CTA-pair (cta_group::2) kernel, forced."""
    torch.manual_seed(3)
    _case(*shape, a_mn, b_mn, impl="pair")


@pytest.mark.parametrize("impl", ["single", "pair"])
def test_epilogues_with_aux_prefetch(impl):
    torch.manual_seed(4)
    _case(1024, 1280, 256, 0, 0, epi=1, alpha=1.0, beta=1.0, impl=impl)      # residual add (bf16 aux)
    _case(1024, 1024, 320, 0, 1, epi=3, impl=impl)                           # ReLU^2 backward
    _case(640, 640, 640, 0, 1, batch=5, epi=1, alpha=0.5, beta=2.0, impl=impl)


@pytest.mark.parametrize("impl", ["single", "pair"])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_split_k_atomic_accumulate(impl, splits):
    from archlab_b200.ops import gemm as G, native

    torch.manual_seed(5)
    M, N, K = 512, 768, 4096
    a = torch.randn(K, M, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    base = torch.randn(M, N, device="cuda")
    out = base.clone()
    G.gemm(a, b, a_mn=True, b_mn=True, out=out, epi=G.EPI_ATOMIC_ADD, impl=impl, splits=splits)
    torch.cuda.synchronize()
    native.check_status()
    ref = base + a.float().t() @ b.float()
    assert ((out - ref).norm() / ref.norm()).item() < 1e-5
