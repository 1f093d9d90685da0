"""Row-sharded frozen FP8 table: a two-rank lookup returns the de-quantised rows of the full table in request order."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import join_ranks


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from archlab_b200.parallel.row_sharded import RowShardedTable, dequantize_rows_e8m0, quantize_rows_e8m0

    torch.manual_seed(0)
    full = torch.randn(37, 64) * torch.logspace(-2, 2, 64)
    table = RowShardedTable(37, 64)
    table.load_full(full)
    assert table.rows == 19 and table.weight.dtype == torch.uint8 and not table.weight.requires_grad
    g = torch.Generator().manual_seed(10 + rank)
    ids = torch.randint(0, 37, (3, 5 + rank), generator=g)          # ranks ask for different numbers of rows
    got = table(ids)
    qv, qe = quantize_rows_e8m0(torch.cat([full, torch.zeros(1, 64)]))
    want = dequantize_rows_e8m0(qv, qe)[ids]
    assert got.shape == (*ids.shape, 64) and got.dtype == torch.bfloat16 and torch.equal(got, want)
    assert ((got.float() - full[ids]).abs() <= full[ids].abs() * 2 ** -4 + 1e-3).all()
    try:
        table(torch.tensor([37]))
        q.put("no error")
    except ValueError:
        q.put("ok")
    # every rank must still be able to take part in a lookup where it asks for nothing
    empty = table(torch.empty(0, dtype=torch.long)) if rank == 0 else table(torch.tensor([1, 20]))
    assert empty.shape[-1] == 64
    dist.destroy_process_group()


def test_two_rank_lookup(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29671, q)) for r in range(2)]
    for p in procs:
        p.start()
    join_ranks(procs, 120)
    assert [q.get(timeout=5) for _ in range(2)] == ["ok", "ok"]


def test_single_process_table_and_width_rule():
    from archlab_b200.parallel.row_sharded import RowShardedTable

    with pytest.raises(ValueError):
        RowShardedTable(8, 48)
    t = RowShardedTable(8, 32)
    t.load_full(torch.arange(8 * 32).float().view(8, 32))
    out = t(torch.tensor([[7, 0]]))
    assert out.shape == (1, 2, 32) and abs(float(out[0, 0, -1]) - 255.0) <= 8
