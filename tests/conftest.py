import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "slow: long-running test")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def join_ranks(procs, timeout: float = 300.0) -> None:
    """Waits for the child processes of a multi-rank test; a rank whose peer failed must not outlive the test
    (it would sit in a collective until the process-group timeout), so stragglers are terminated."""
    try:
        for p in procs:
            p.join(timeout=timeout)
            assert not p.is_alive(), "worker timed out"
            assert p.exitcode == 0, f"worker exited with code {p.exitcode}"
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=30)
