"""Node-local groups: layout rules on one machine, group creation on a 4-rank gloo job with faked host names."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from archlab_b200.parallel.node_groups import group_layout, ranks_per_host
from conftest import join_ranks


def test_layout_rules():
    hosts = ["a", "a", "a", "a", "b", "b", "b", "b"]
    assert group_layout(hosts, 4) == [[0, 1, 2, 3], [4, 5, 6, 7]] and group_layout(hosts, 2)[2] == [4, 5]
    with pytest.raises(ValueError, match="must divide"):
        group_layout(hosts, 3)
    with pytest.raises(ValueError, match="span hosts"):
        group_layout(hosts, 8)
    with pytest.raises(ValueError, match="span hosts"):
        group_layout(["a", "b", "a", "b"], 2)
    assert ranks_per_host(["a", "b", "a"]) == {"a": [0, 2], "b": [1]}


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from archlab_b200.parallel.node_groups import node_local_groups

        group, ranks = node_local_groups(2, host_of=lambda: f"host-{rank // 2}")
        assert ranks == [2 * (rank // 2), 2 * (rank // 2) + 1]
        t = torch.tensor([float(rank)])
        dist.all_reduce(t, group=group)
        assert float(t) == sum(ranks)
        try:
            node_local_groups(2, host_of=lambda: f"host-{rank % 2}")               # interleaved hosts: every rank refuses
            raise AssertionError("a cross-host group was accepted")
        except ValueError as error:
            assert "span hosts" in str(error)
    finally:
        dist.destroy_process_group()


def test_groups_on_four_ranks():
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 4, 29671)) for r in range(4)]
    for p in procs:
        p.start()
    join_ranks(procs)
