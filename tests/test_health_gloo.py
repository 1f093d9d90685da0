"""Failure detection on host ranks: non-finite loss on one rank stops all, stop requests reach consensus,
a rank that never joins fails the probe within its timeout, diverged ranks are caught."""
import json
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, run_dir, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from archlab_b200.train import health as H

        res = {"probe": H.collective_probe()["world_size"]}
        guard = H.FiniteGuard()
        guard.check(0, 1.0, 2.0)
        try:
            guard.check(1, float("nan") if rank == 1 else 1.0)
            res["finite"] = "missed"
        except FloatingPointError:
            res["finite"] = "raised"                               # on BOTH ranks, though only rank 1 saw the NaN
        stop = H.StopConsensus(run_dir, install_signals=False)
        res["stop0"] = stop.should_stop()
        if rank == 1:
            stop.requested, stop.reason = True, "test"             # as a signal handler would
        res["stop1"] = stop.should_stop()
        stop.acknowledge(7, rank)
        H.assert_ranks_agree("weights", H.digest_tensors([torch.ones(3)]))
        try:
            H.assert_ranks_agree("cursor", H.digest_tensors([torch.full((2,), float(rank))]))
            res["agree"] = "missed"
        except RuntimeError:
            res["agree"] = "raised"
        out[rank] = res
    finally:
        dist.destroy_process_group()


def test_detection_and_stop_consensus(tmp_path):
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), out), nprocs=2, join=True)
        for r in (0, 1):
            assert out[r] == {"probe": 2, "finite": "raised", "stop0": False, "stop1": True, "agree": "raised"}
    assert json.loads((tmp_path / "STOPPED.json").read_text())["step"] == 7


def _absent_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from archlab_b200.train import health as H

    if rank == 1:
        time.sleep(6)                                              # "never joins": sleeps through the probe window, then exits
        out[rank] = "absent"
        return
    t0 = time.time()
    try:
        H.collective_probe(timeout_seconds=2.0)
        out[rank] = "passed"
    except Exception as e:                                         # noqa: BLE001 - any backend error is the signal
        out[rank] = f"failed after {time.time() - t0:.0f}s"


def test_probe_fails_fast_when_a_rank_never_joins():
    with mp.Manager() as mgr:
        out = mgr.dict()
        try:
            mp.spawn(_absent_worker, args=(2, _free_port(), out), nprocs=2, join=True)
        except Exception:                                          # the surviving rank may exit non-zero at teardown
            pass
        assert out.get(0, "").startswith("failed") and int(out[0].split()[2][:-1]) <= 5


def test_heartbeat_and_stop_file(tmp_path):
    from archlab_b200.train import health as H

    hb = H.Heartbeat(tmp_path, period=0.05)
    assert hb.beat(step=1) and not hb.beat(step=2)
    time.sleep(0.06)
    assert hb.beat(step=3) and json.loads((tmp_path / "HEARTBEAT.json").read_text())["step"] == 3
    stop = H.StopConsensus(tmp_path, install_signals=False)
    assert not stop.should_stop()
    (tmp_path / "STOP_REQUESTED.json").write_text("{}")
    assert stop.should_stop() and stop.reason == "STOP_REQUESTED.json"
    with pytest.raises(FloatingPointError):
        H.FiniteGuard().check(3, float("inf"))
