"""A bounded device wait that runs out: the barrier kernel waits for a flag that nothing sets, gives up after its
(shortened) budget, returns, and reports through the status word; the context stays usable afterwards.  No peer is
involved: both entries of the pointer table are local arrays, one standing in for the other rank's."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_barrier_wait_expires_and_reports_operational_failure():
    from archlab_b200.contracts.substrate import classify_failure
    from archlab_b200.ops import native
    from archlab_b200.parallel import symm  # noqa: F401  (registers the barrier's signature)

    L = native.lib()
    L.nga_set_peer_wait_budget_ns.argtypes, L.nga_set_peer_wait_budget_ns.restype = [C.c_ulonglong], None
    L.nga_peer_wait_budget_ns.restype = C.c_ulonglong
    default = L.nga_peer_wait_budget_ns()
    assert default == 30_000_000_000                                # inter-GPU waits tolerate a late rank by default
    mine = torch.zeros(16, dtype=torch.int32, device="cuda")       # this rank's flag array
    other = torch.zeros(16, dtype=torch.int32, device="cuda")      # stands in for rank 1's; rank 1 never runs
    table = (C.c_longlong * 2)(mine.data_ptr(), other.data_ptr())
    status = native.status_word()
    status.zero_()
    L.nga_set_peer_wait_budget_ns(20_000_000)                      # 20 ms
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = L.nga_peer_barrier(table, 0, 2, 1, status.data_ptr(), native.stream_ptr())
        t1.record()
        assert rc == 0
        torch.cuda.synchronize()                                   # returns: the wait is bounded
        assert 15.0 < t0.elapsed_time(t1) < 1000.0
        assert int(mine[0]) == 1 and int(other[0]) == 1 and int(mine[1]) == 0
        assert int(status.item()) == 2
        with pytest.raises(native.NativeError) as err:
            native.check_status()
        assert classify_failure(err.value).category == "operational"
        assert int(status.item()) == 0                             # check_status cleared the word
    finally:
        L.nga_set_peer_wait_budget_ns(0)
    assert L.nga_peer_wait_budget_ns() == default
    # the context is alive: a satisfied barrier (the stand-in flag now set by hand) passes without a report
    mine[1] = 2
    rc = L.nga_peer_barrier(table, 0, 2, 2, status.data_ptr(), native.stream_ptr())
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0
