"""Shared model blocks: norms, rotary variants, hyper-connections, hashed memories."""
import math

import torch

from archlab_b200.models import blocks as bk


def test_group_rms_norm_is_per_stream():
    n = bk.GroupRMSNorm(8, 3, zero_centered=True)
    x = torch.randn(2, 5, 24)
    y = n(x).unflatten(-1, (3, 8))
    torch.testing.assert_close(y.square().mean(-1), torch.ones(2, 5, 3), atol=1e-4, rtol=1e-4)
    n2 = bk.GroupRMSNorm(8, 3)
    torch.testing.assert_close(n2(x), n(x))


def test_rope_styles_preserve_norm_and_partial_passthrough():
    x = torch.randn(2, 6, 3, 16)
    cos, sin = bk.rope_tables(6, 8)
    for style in ("half", "interleaved"):
        y = bk.apply_rope(x, cos, sin, style=style, rot_dim=8)
        torch.testing.assert_close(y[..., 8:], x[..., 8:])
        torch.testing.assert_close(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(y[:, 0], x[:, 0])      # position 0 is the identity


def test_so3_rope_keeps_determinants_at_equal_positions():
    a, b, c = (torch.randn(4, 1, 9) for _ in range(3))
    pos = torch.tensor([0.0, 1.0, 5.0, 17.0])[:, None]
    ra, rb, rc = (bk.so3_chunk_rope(t, pos) for t in (a, b, c))
    det = lambda u, v, w: torch.linalg.det(torch.stack([u.unflatten(-1, (3, 3)), v.unflatten(-1, (3, 3)),
                                                         w.unflatten(-1, (3, 3))], -1))
    torch.testing.assert_close(det(ra, rb, rc), det(a, b, c), atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(ra.norm(dim=-1), a.norm(dim=-1), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(ra[0], a[0])


def test_sinkhorn_maps_are_doubly_stochastic():
    m = bk.sinkhorn_knopp(torch.randn(7, 4, 4), 30)
    torch.testing.assert_close(m.sum(-2), torch.ones(7, 4), atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(m.sum(-1), torch.ones(7, 4), atol=1e-3, rtol=1e-3)
    pre, post, comb = bk.hc_split_sinkhorn(torch.randn(5, 24), torch.tensor([0.5, 0.5, 0.5]), torch.zeros(24))
    assert pre.shape == (5, 4) and post.shape == (5, 4) and comb.shape == (5, 4, 4)
    assert (pre > 0).all() and (post < 2).all()
    torch.testing.assert_close(comb.sum(-2), torch.ones(5, 4), atol=1e-3, rtol=1e-3)


def test_hyper_connection_roundtrip_shapes_and_grad():
    hc = bk.HyperConnection(16, 4)
    hc.init_weights()
    s = torch.randn(2, 3, 4, 16, requires_grad=True)
    x, post, res = hc.prepare(s)
    assert x.shape == (2, 3, 16)
    out = hc.combine(s, x * 2, post, res)
    assert out.shape == s.shape
    out.sum().backward()
    assert s.grad is not None and hc.mapping_proj.weight.grad is not None


def test_gated_stream_residual_inject():
    gr = bk.GatedStreamResidual(8, 4, low_rank=4)
    packed = torch.randn(2, 3, 32)
    mixed, same, w = gr(packed)
    assert mixed.shape == (2, 3, 8) and w.shape == (2, 3, 4) and same is packed
    out = gr.inject(packed, torch.ones(2, 3, 8), w)
    torch.testing.assert_close((out - packed).unflatten(-1, (4, 8))[..., 0], w)


def test_prime_sizes_and_hash_segments():
    sizes = bk.distinct_prime_sizes(100, 4, divisor=8)
    assert len(set(sizes)) == 4 and sum(sizes) % 8 == 0 and all(bk._is_prime(s) for s in sizes)
    mult = bk.hash_multipliers(1000, 3)
    assert (mult % 2 == 1).all() and (mult * 1000 > 0).all()
    h = bk.NgramHash(1000, 3, 2, [101, 103, 107, 109], eos=0)
    t = torch.tensor([[5, 6, 0, 7, 8, 9]])
    ids = h(t)
    assert ids.shape == (1, 6, 4)
    # the token right after EOS sees EOS as its history: same ids as a sequence that starts there
    ids2 = h(torch.tensor([[7, 8, 9]]))
    assert torch.equal(ids[0, 3:], ids2[0])
    lo = torch.tensor([0, 101, 204, 311])
    assert ((ids >= lo) & (ids < lo + torch.tensor([101, 103, 107, 109]))).all()


def test_owner_sharded_embedding_single_owner_matches_dense_table():
    emb = bk.OwnerShardedEmbedding(4, 10, 6)
    emb.reset_parameters()
    ids = torch.randint(0, 40, (3, 7))
    dense = torch.cat([t.view(10, 6) for t in emb.tables])
    torch.testing.assert_close(emb(ids), dense[ids])


def test_engram_memory_shapes():
    m = bk.EngramMemory(hidden=16, memory_dim=8, vocab=50, heads=2, orders=(2, 3))
    x = torch.randn(2, 9, 16)
    ids = torch.randint(0, 50, (2, 9))
    y = m(x, ids, pad_id=0)
    assert y.shape == x.shape and torch.isfinite(y).all()
    # changing a token only affects positions whose n-gram window covers it
    ids2 = ids.clone()
    ids2[:, 6] = (ids2[:, 6] + 1) % 50
    y2 = m(x, ids2, pad_id=0)
    torch.testing.assert_close(y[:, :6], y2[:, :6])
