"""Triadic GDN, local attention and LinSimp oracles on CPU."""
import torch

from archlab_b200.ops import linsimp, local_attention as la, triadic


def _tri_inputs(B=2, T=70, H=2, D=8, E=3, V=8, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=dtype)
    q, k, v = r(B, T, H, D) * 0.5, r(B, T, H, D) * 0.5, r(B, T, H, V)
    k2, q2 = r(B, T, H, E) * 0.5, r(B, T, H, E) * 0.5
    gg = -torch.rand(B, T, H, E, generator=g, dtype=dtype) * 0.2
    beta = torch.rand(B, T, H, generator=g, dtype=dtype)
    return q, k, v, k2, q2, gg, beta


def test_triadic_chunked_matches_recurrence():
    args = _tri_inputs()
    ref = triadic.triadic_gdn_reference(*args)
    out = triadic.triadic_gdn_attention(*args)
    torch.testing.assert_close(out, ref, atol=2e-5, rtol=1e-4)


def test_triadic_packed_documents_reset_state():
    args = _tri_inputs(B=1, T=50)
    cu = torch.tensor([0, 20, 50])
    packed = triadic.triadic_gdn_attention(*args, cu_seqlens=cu)
    second = triadic.triadic_gdn_reference(*[t[:, 20:] for t in args])
    torch.testing.assert_close(packed[:, 20:], second, atol=2e-5, rtol=1e-4)
    # E = 1 with k2 = q2 = 1 is the ordinary gated delta rule (without q/k normalisation)
    q, k, v, k2, q2, g, beta = _tri_inputs(E=1)
    one = torch.ones_like(k2)
    a = triadic.triadic_gdn_reference(q, k, v, one, one, g, beta)
    b = triadic.triadic_gdn_attention(q, k, v, one, one, g, beta)
    torch.testing.assert_close(a, b, atol=2e-5, rtol=1e-4)


def test_local_attention_window_semantics():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 12, 4, 8), torch.randn(1, 12, 2, 8), torch.randn(1, 12, 2, 8)
    full = la.reference_local_attention(q, k, v, 12)
    sdpa = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.repeat_interleave(2, 2).transpose(1, 2), v.repeat_interleave(2, 2).transpose(1, 2),
        is_causal=True).transpose(1, 2)
    torch.testing.assert_close(full, sdpa, atol=1e-5, rtol=1e-5)
    one = la.local_attention(q, k, v, 1)                       # window 1: every query reads itself only
    torch.testing.assert_close(one, v.repeat_interleave(2, 2))


def test_linsimp_vectorised_matches_loop_and_rf_limit():
    torch.manual_seed(0)
    B, T, H, D = 2, 10, 2, 4
    q, k, r, v, u = (torch.randn(B, T, H, D) for _ in range(5))
    omega = linsimp.orthogonal_feature_bank(H, D, 8)
    assert omega.shape == (H, 8, D)
    a = linsimp.linsimp_attention(q, k, r, v, u, omega, window=3)
    b = linsimp.linsimp_attention_loop(q, k, r, v, u, omega, window=3)
    torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-4)
    # causal: changing a future token leaves earlier outputs untouched
    v2 = v.clone()
    v2[:, 7:] += 1
    torch.testing.assert_close(linsimp.linsimp_attention(q, k, r, v2, u, omega, window=3)[:, :7], a[:, :7])
    out = linsimp.linear_rf_attention(q, k, v, omega)
    assert out.shape == q.shape and torch.isfinite(out).all()
