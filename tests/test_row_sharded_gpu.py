"""Owner-side gather + de-quantisation kernel of the row-sharded FP8 tables against its PyTorch statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,dim,n", [(1000, 256, 4096), (37, 64, 11), (50000, 1280, 20000)])
def test_gather_dequant_matches_torch(rows, dim, n):
    from archlab_b200.ops import native
    from archlab_b200.parallel.row_sharded import RowShardedTable, dequantize_rows_e8m0

    torch.manual_seed(0)
    table = RowShardedTable(rows, dim, device="cuda")
    table.load_full(torch.randn(rows, dim) * torch.logspace(-3, 3, dim))
    ids = torch.randint(0, rows, (n,), device="cuda")
    got = table(ids)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(got, dequantize_rows_e8m0(table.weight[ids], table.scale[ids]))
