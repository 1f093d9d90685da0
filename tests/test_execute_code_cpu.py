"""Grading generated programs: success, failure with the last error line, timeout, memory."""
import pytest

from archlab_b200.train.local_sandbox import execute_code, strongest_isolation

ALLOW = strongest_isolation() == "rlimits"


def test_outcomes_are_classified():
    ok = execute_code("def add(a, b):\n    return a + b\nassert add(2, 3) == 5\nprint('passed')", allow_unisolated=ALLOW)
    assert ok.success and ok.stdout.strip() == "passed" and ok.error is None
    wrong = execute_code("def add(a, b):\n    return a - b\nassert add(2, 3) == 5", allow_unisolated=ALLOW)
    assert not wrong.success and "AssertionError" in wrong.error and not wrong.timeout
    slow = execute_code("while True:\n    pass", timeout=1.0, allow_unisolated=ALLOW)
    assert not slow.success and slow.timeout and slow.error == "execution timed out"
    big = execute_code("x = bytearray(2 * 1024 ** 3)", memory_mb=256, allow_unisolated=ALLOW)
    assert not big.success and big.memory_exceeded and big.error == "memory limit exceeded"
    crash = execute_code("import sys\nsys.exit(3)", allow_unisolated=ALLOW)
    assert not crash.success and crash.error == "exit code 3"
