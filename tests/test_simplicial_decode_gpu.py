"""Paged simplicial decode on the tcgen05 kernel against the fp32 statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("Hq,Hkv,w1,w2,lens", [(4, 1, 32, 512, [700, 129, 40]), (8, 2, 16, 128, [300, 128]), (2, 2, 8, 64, [5, 1000])])
def test_paged_decode_kernel(Hq, Hkv, w1, w2, lens):
    from archlab_b200.ops import native
    from archlab_b200.ops.simplicial_decode import PagedSimplicialCache, simplicial_decode, simplicial_decode_reference

    torch.manual_seed(0)
    D = 128
    cache = PagedSimplicialCache(24, Hkv, D, "cuda")
    for t in (cache.k1, cache.k2, cache.v1, cache.v2):
        t.normal_()                                          # stale rows must be masked, not relied on to be zero
    perm = torch.randperm(24).tolist()
    cache.free = perm                                        # scattered physical pages
    tables = []
    for L in lens:
        pages = torch.tensor(cache.allocate(L), device="cuda")
        mk = lambda: (torch.randn(L, Hkv, D, device="cuda") * 0.7).bfloat16()
        cache.write(pages, 0, mk(), mk(), mk(), mk())
        tables.append(torch.nn.functional.pad(pages, (0, 8 - pages.numel())))
    q = (torch.randn(len(lens), Hq, D, device="cuda") * 0.7).bfloat16()
    bt, sl = torch.stack(tables).int(), torch.tensor(lens, device="cuda", dtype=torch.int32)
    got = simplicial_decode(q, cache, bt, sl, w1, w2)
    torch.cuda.synchronize()
    native.check_status()
    want = simplicial_decode_reference(q, cache, bt, sl, w1, w2)
    assert (got.float() - want).norm() / want.norm() < 2e-2
