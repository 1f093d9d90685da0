"""Selected-key sink attention on the flash kernels against the gather-based fp32 statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("top_k", [None, 96])
def test_selected_sink_attention_forward_backward(top_k):
    from archlab_b200.ops import dsa, dsa_cuda, native

    torch.manual_seed(0)
    B, T, H, D = 2, 256, 4, 128
    q = (torch.randn(B, T, H, D, device="cuda") * 0.6).bfloat16().requires_grad_(True)
    kv = (torch.randn(B, T, D, device="cuda") * 0.6).bfloat16().requires_grad_(True)
    sink = (torch.randn(H, device="cuda") * 0.5).requires_grad_(True)
    idx = None
    if top_k is not None:
        scores = torch.randn(B, T, T, device="cuda")
        scores = scores.masked_fill(torch.arange(T, device="cuda")[None, :] > torch.arange(T, device="cuda")[:, None], float("-inf"))
        idx, _ = dsa.select_topk(scores, top_k)
    w = torch.randn(B, T, H, D, device="cuda")
    o = dsa_cuda.selected_sink_attention(q, kv, sink, idx)
    (o.float() * w).sum().backward()
    native.check_status()
    qf, kvf, sf = (t.detach().float().requires_grad_(True) for t in (q, kv, sink))
    scale = D ** -0.5
    ref = dsa.dense_sink_attention(qf, kvf, sf, scale) if idx is None else dsa.sparse_attention(qf, kvf, sf, idx, scale, recompute=False)
    (ref * w).sum().backward()
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()
    assert rel(o, ref) < 2e-2
    assert rel(q.grad, qf.grad) < 3e-2 and rel(kv.grad, kvf.grad) < 3e-2 and rel(sink.grad, sf.grad) < 3e-2


@pytest.mark.parametrize("S,top_k", [(256, 64), (1024, 512), (96, 200)])
def test_indexer_selection_kernel_matches_topk_threshold(S, top_k):
    from archlab_b200.ops import dsa, dsa_cuda, native

    torch.manual_seed(1)
    B = 2
    q = torch.randn(B, S, 4, 64, device="cuda").bfloat16()
    k = torch.randn(B, S, 64, device="cuda").bfloat16()
    w = torch.rand(B, S, 4, device="cuda")
    bits, bits_t = dsa_cuda.indexer_select(q, k, w, top_k)
    torch.cuda.synchronize()
    native.check_status()
    scores = dsa.indexer_scores(q, k, w)
    idx, vals = dsa.select_topk(scores, top_k)
    want, want_t = dsa_cuda.selection_bits_from_scores(scores, vals[..., -1:])
    # scores are recomputed in a different summation order: allow the few keys that sit on the threshold to differ
    # (exact ties, e.g. keys whose four head products are all negative and score 0, are selected together by both)
    unpack = lambda t: torch.stack([(t.view(torch.uint8) >> i) & 1 for i in range(8)], -1).flatten(-2)[..., :S].bool()
    got, ref = unpack(bits), unpack(want)
    flipped = int((got ^ ref).sum())
    assert flipped <= 0.002 * B * S * S, flipped
    assert torch.equal(bits_t, dsa_cuda.transpose_bits(bits, S)) and torch.equal(unpack(bits_t), got.transpose(1, 2))
    rows = torch.arange(S, device="cuda")
    assert not (got & (rows[None, :] > rows[:, None])[None]).any()                    # nothing above the diagonal
    assert torch.all(got.sum(-1) >= torch.clamp(rows + 1, max=top_k)[None, :])        # at least k (all, when fewer exist)
    assert (got.sum(-1) - ref.sum(-1)).abs().max() <= 4
