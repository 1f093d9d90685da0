"""Process sandbox for agent tools: run an untrusted snippet with a time limit, a scrubbed environment and a
private working directory, and verify a task by running its checker in the same directory.

The reference reaches E2B or a rootless-namespace pod for this (src/archlab/training/sandbox.py,
dlc_sandbox.py); on a single box a subprocess with resource limits is the equivalent boundary used by the
agent-tool gate.  Nothing is inherited from the caller's environment except PATH.
"""
from __future__ import annotations

import os
import resource
import subprocess
import sys
import tempfile
from dataclasses import dataclass
from pathlib import Path


@dataclass(frozen=True)
class ToolResult:
    returncode: int
    stdout: str
    stderr: str
    timed_out: bool


class LocalSandbox:
    def __init__(self, *, cpu_seconds: int = 5, memory_mb: int = 512, wall_seconds: float = 10.0):
        self.cpu, self.mem, self.wall = cpu_seconds, memory_mb, wall_seconds
        self._dir = tempfile.TemporaryDirectory(prefix="archlab-sandbox-")
        self.root = Path(self._dir.name)

    def _limits(self):
        resource.setrlimit(resource.RLIMIT_CPU, (self.cpu, self.cpu))
        resource.setrlimit(resource.RLIMIT_AS, (self.mem << 20, self.mem << 20))
        resource.setrlimit(resource.RLIMIT_NPROC, (64, 64))
        os.setsid()

    def write(self, name: str, text: str) -> Path:
        p = (self.root / name).resolve()
        if self.root.resolve() not in p.parents:
            raise ValueError("path escapes the sandbox")
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(text)
        return p

    def run_python(self, code: str, *, stdin: str = "") -> ToolResult:
        script = self.write("_tool.py", code)
        try:
            r = subprocess.run([sys.executable, "-I", str(script)], cwd=self.root, input=stdin, capture_output=True, text=True,
                               timeout=self.wall, env={"PATH": os.environ.get("PATH", "")}, preexec_fn=self._limits)
            return ToolResult(r.returncode, r.stdout[-8192:], r.stderr[-8192:], False)
        except subprocess.TimeoutExpired as e:
            return ToolResult(-9, (e.stdout or b"").decode(errors="replace")[-8192:] if isinstance(e.stdout, bytes) else (e.stdout or ""),
                              "", True)

    def verify(self, checker_code: str) -> bool:
        """The checker runs in the sandbox directory (it can read files the tools wrote); exit code 0 = solved."""
        r = self.run_python(checker_code)
        return r.returncode == 0 and not r.timed_out

    def close(self) -> None:
        self._dir.cleanup()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
