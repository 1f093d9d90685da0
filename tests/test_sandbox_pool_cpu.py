"""Sandbox pool over HTTP: capacity refusals, expiry, timeouts as code 124, transport errors that are never verdicts."""
import threading

import pytest

from archlab_b200.train import sandbox_pool as sp
from archlab_b200.train.local_sandbox import LocalSandbox, strongest_isolation


def _sandbox(image):
    if strongest_isolation() == "rlimits":
        return LocalSandbox(wall_seconds=2.0, isolation="rlimits", allow_unisolated=True)
    return LocalSandbox(wall_seconds=2.0)


@pytest.fixture()
def service(tmp_path):
    now = [0.0]
    pool = sp.Pool(2, _sandbox, lifetime=100.0, clock=lambda: now[0])
    server = sp.make_server(pool)
    thread = threading.Thread(target=server.serve_forever, daemon=True)
    thread.start()
    sp.announce(tmp_path / "pool", server, 2)
    yield pool, tmp_path / "pool", now
    server.shutdown()
    server.server_close()


def test_round_trip_capacity_and_expiry(service):
    pool, pool_dir, now = service
    a = sp.SandboxClient(pool_dir, capacity_wait_seconds=0.2, retry_seconds=0.05)
    a.start("image-a")
    a.copy_to("data/in.txt", "41")
    out = a.execute("print(int(open('data/in.txt').read()) + 1)")
    assert out["returncode"] == 0 and out["stdout"].strip() == "42" and not out["timed_out"]
    assert a.execute("raise SystemExit(3)")["returncode"] == 3
    slow = a.execute("import time\nprint('partial', flush=True)\ntime.sleep(30)")
    assert slow["returncode"] == sp.TIMEOUT_CODE and slow["timed_out"]
    b = sp.SandboxClient(pool_dir, capacity_wait_seconds=0.2, retry_seconds=0.05)
    b.start("image-b")
    c = sp.SandboxClient(pool_dir, capacity_wait_seconds=0.2, retry_seconds=0.05)
    with pytest.raises(sp.TransportError, match="no sandbox capacity"):
        c.start("image-c")
    assert pool.health() == {"slots": 2, "busy": 2}
    now[0] = 101.0                                                      # both clients "vanished": their slots come back
    c.start("image-c")
    assert pool.health()["busy"] == 1
    with pytest.raises(sp.TransportError, match="answered 404"):
        a.execute("print(1)")
    c.cleanup()
    assert pool.health()["busy"] == 0
    with pytest.raises(sp.TransportError, match="answered 400"):
        d = sp.SandboxClient(pool_dir)
        d.start("image-d")
        d.copy_to("../escape.txt", "x")


def test_unreachable_servers_raise_transport_errors(tmp_path):
    with pytest.raises(sp.TransportError, match="no sandbox server announced"):
        sp.SandboxClient(tmp_path).start("x")
    (tmp_path / "dead.json").write_text('{"url": "http://127.0.0.1:9", "slots": 1}')
    with pytest.raises(sp.TransportError, match="reachable"):
        sp.SandboxClient(tmp_path, capacity_wait_seconds=0.1, request_timeout=0.5).start("x")
    urls = [f"http://h{i}:1" for i in range(6)]
    assert sp.affinity_order("img", urls) == sp.affinity_order("img", list(reversed(urls))) != sp.affinity_order("other", urls)
    with pytest.raises(RuntimeError, match="start the sandbox first"):
        sp.SandboxClient(tmp_path).execute("print(1)")
