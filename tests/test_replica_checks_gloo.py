"""Unique-parameter counting and replica equality on a 4-rank gloo job (2 expert shards x 2 replicas)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import join_ranks


def _worker(rank, world, port, diverge):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from archlab_b200.train.replica_checks import effective_gradient, replica_equality, unique_parameter_counts

        torch.manual_seed(0)
        model = torch.nn.Module()
        model.dense = torch.nn.Linear(8, 8, bias=False)                       # same on every rank
        torch.manual_seed(100 + rank % 2)                                     # expert shard r % 2; ranks r and r + 2 are replicas
        model.experts = torch.nn.Linear(8, 6, bias=False)
        model.experts.weight.allreduce = False
        groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
        counts = unique_parameter_counts(model, data_replicas=4, expert_replicas=2)
        assert counts == {"dense_unique": 64, "expert_side_unique": 96, "total": 160}, counts
        try:
            unique_parameter_counts(model, data_replicas=3, expert_replicas=2)
            raise AssertionError("indivisible replica count accepted")
        except RuntimeError:
            pass
        if diverge and rank == 3:
            with torch.no_grad():
                model.experts.weight[0, 0] += 1
        try:
            report = replica_equality(model, groups[rank % 2], ("experts.",))
            assert not diverge and report["checked_tensors_all_ranks"] == 4
        except RuntimeError as error:
            assert diverge and "replica equality failed" in str(error)
        try:
            replica_equality(model, groups[rank % 2], ("no_such_module.",))
            raise AssertionError("vacuous check passed")
        except RuntimeError:
            pass
        p = model.dense.weight
        p.main_grad, p.grad_added_to_main_grad = torch.ones_like(p), True
        assert effective_gradient(p, None) is p.main_grad and effective_gradient(model.experts.weight, "g") == "g"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("diverge", [False, True])
def test_replica_checks(diverge):
    port = 29650 + int(diverge)
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 4, port, diverge)) for r in range(4)]
    for p in procs:
        p.start()
    join_ranks(procs)
