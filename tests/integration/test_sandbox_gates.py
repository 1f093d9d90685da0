"""Sandbox gate: an agent tool call runs isolated, and a task verifier accepts a correct solution only."""
import os

from archlab_b200.train.local_sandbox import LocalSandbox


def test_agent_tool_and_successful_verifier():
    with LocalSandbox(wall_seconds=10) as sb:
        r = sb.run_python("import os\nopen('answer.txt', 'w').write(str(sum(range(101))))\nprint(sorted(os.environ))")
        assert r.returncode == 0 and "HOME" not in r.stdout and "PATH" in r.stdout
        checker = "import sys\nsys.exit(0 if open('answer.txt').read().strip() == '5050' else 1)"
        assert sb.verify(checker)
        sb.write("answer.txt", "41")
        assert not sb.verify(checker)
        slow = sb.run_python("while True: pass")
        assert slow.timed_out or slow.returncode != 0
        try:
            sb.write("../escape.txt", "x")
            raise AssertionError("path escape must be refused")
        except ValueError:
            pass


def test_a_forked_grandchild_does_not_outlive_the_timeout():
    import os
    import time

    with LocalSandbox(wall_seconds=2, cpu_seconds=30) as sb:
        code = ("import os, time\n"
                "pid = os.fork()\n"
                "if pid == 0:\n"
                "    open('child.pid', 'w').write(str(os.getpid()))\n"
                "    time.sleep(60)\n"
                "    os._exit(0)\n"
                "time.sleep(60)\n")
        t0 = time.time()
        r = sb.run_python(code)
        assert r.timed_out and time.time() - t0 < 15
        if sb.isolation == "namespaces":
            return          # pids inside a PID namespace are not this process's; --kill-child ends the namespace
        pid = int((sb.root / "child.pid").read_text())
        for _ in range(50):
            try:
                os.kill(pid, 0)
            except ProcessLookupError:
                break
            time.sleep(0.1)
        else:
            raise AssertionError("grandchild survived the sandbox timeout")


def test_grandchild_is_killed_without_namespaces_too():
    import os
    import time

    mode = "uid" if os.geteuid() == 0 else "rlimits"
    with LocalSandbox(wall_seconds=2, cpu_seconds=30, isolation=mode, allow_unisolated=True) as sb:
        r = sb.run_python("import os, time\n"
                          "if os.fork() == 0:\n"
                          "    open('child.pid', 'w').write(str(os.getpid()))\n"
                          "    time.sleep(60)\n"
                          "    os._exit(0)\n"
                          "time.sleep(60)\n")
        assert r.timed_out
        pid = int((sb.root / "child.pid").read_text())
        deadline = time.time() + 5
        while time.time() < deadline:
            try:
                os.kill(pid, 0)
            except ProcessLookupError:
                return
            time.sleep(0.1)
        raise AssertionError("grandchild survived the sandbox timeout")


def test_isolation_is_reported_and_resource_limits_alone_are_refused():
    import pytest

    from archlab_b200.train.local_sandbox import SandboxUnavailable, strongest_isolation

    with pytest.raises(SandboxUnavailable):
        LocalSandbox(isolation="rlimits")
    with LocalSandbox(wall_seconds=10) as sb:
        assert sb.isolation == strongest_isolation()
        r = sb.run_python("import os\nprint(os.geteuid())\n"
                          "import socket\ns = socket.socket()\ns.settimeout(1)\n"
                          "try:\n    s.connect(('1.1.1.1', 53)); print('net')\nexcept OSError:\n    print('nonet')\n")
        assert r.returncode == 0, r.stderr
        uid, net = r.stdout.split()
        if sb.isolation == "namespaces":
            assert net == "nonet"
        if sb.isolation in ("namespaces", "uid") and os.geteuid() == 0:
            assert uid != "0"

