"""Paged decode statement equals the last row of the full windowed simplicial attention."""
import torch

from archlab_b200.ops import simplicial as sx
from archlab_b200.ops.simplicial_decode import PagedSimplicialCache, simplicial_decode


def test_paged_decode_matches_full_attention_last_row():
    torch.manual_seed(0)
    Hq, Hkv, D, w1, w2 = 4, 2, 16, 4, 150
    cache = PagedSimplicialCache(6, Hkv, D, "cpu", torch.float32)
    lens = [200, 131]
    tables, qs, wants = [], [], []
    for L in lens:
        q, k1, k2, v1, v2 = (torch.randn(1, L, h, D) for h in (Hq, Hkv, Hkv, Hkv, Hkv))
        pages = torch.tensor(cache.allocate(L))
        cache.write(pages, 0, k1[0], k2[0], v1[0], v2[0])
        tables.append(torch.nn.functional.pad(pages, (0, 3 - pages.numel())))
        qs.append(q[0, -1])
        wants.append(sx.simplicial_attention_reference(q, k1, k2, v1, v2, w1, w2)[0, -1])
    got = simplicial_decode(torch.stack(qs), cache, torch.stack(tables), torch.tensor(lens), w1, w2)
    assert torch.allclose(got, torch.stack(wants), atol=1e-5)
    cache.release(tables[0][:2].tolist())
    assert len(cache.free) == 4
