"""Process sandbox for agent tools: run an untrusted snippet with a time limit, a scrubbed environment and a
private working directory, and verify a task by running its checker in the same directory.

The reference reaches E2B or a rootless-namespace pod for this (src/archlab/training/sandbox.py,
dlc_sandbox.py).  On a single box the child runs in the strongest isolation the host offers, probed once:

``namespaces``  ``unshare`` with new network, PID and mount namespaces (no network, no view of other processes,
                killed as a unit when the namespace's init exits).  A root caller also drops the child to
                ``nobody`` inside them; a rootless caller gets them through a user namespace and the child keeps
                the caller's file permissions.
``uid``         no namespaces, but the caller is root: the child runs as ``nobody`` (so ``RLIMIT_NPROC`` binds and
                the caller's files are not writable); the network stays reachable.
``rlimits``     resource limits only.  This is **not a security boundary**: the snippet runs as the caller with the
                caller's filesystem and network.  It is refused unless ``allow_unisolated=True`` is passed.

In every mode the child gets CPU / address-space / process-count limits, its own session, and the whole
process group is killed when the wall-clock limit expires, so a forked grandchild does not outlive the call.
Nothing is inherited from the caller's environment except PATH.
"""
from __future__ import annotations

import functools
import os
import resource
import shutil
import signal
import subprocess
import sys
import tempfile
from dataclasses import dataclass
from pathlib import Path

NOBODY = 65534


class SandboxUnavailable(RuntimeError):
    """No isolation stronger than resource limits exists on this host and none was waived."""


@dataclass(frozen=True)
class ToolResult:
    returncode: int
    stdout: str
    stderr: str
    timed_out: bool


@functools.lru_cache(maxsize=1)
def namespace_command() -> tuple[str, ...] | None:
    """The ``unshare`` prefix that works here, or None."""
    exe = shutil.which("unshare")
    if exe is None:
        return None
    common = ("--net", "--pid", "--fork", "--mount-proc", "--kill-child")
    if os.geteuid() == 0:       # real namespaces, then an unprivileged uid inside them
        cmd = (exe, *common, "--setgid", str(NOBODY), "--setuid", str(NOBODY))
    else:                       # rootless: a user namespace carries the others; files stay those of the caller
        cmd = (exe, "--user", "--map-root-user", *common)
    try:
        ok = subprocess.run([*cmd, "true"], capture_output=True, timeout=10).returncode == 0
    except (OSError, subprocess.TimeoutExpired):
        ok = False
    return cmd if ok else None


def strongest_isolation() -> str:
    if namespace_command() is not None:
        return "namespaces"
    return "uid" if os.geteuid() == 0 else "rlimits"


class LocalSandbox:
    def __init__(self, *, cpu_seconds: int = 5, memory_mb: int = 512, wall_seconds: float = 10.0,
                 max_processes: int = 64, isolation: str = "auto", allow_unisolated: bool = False):
        self.cpu, self.mem, self.wall, self.nproc = cpu_seconds, memory_mb, wall_seconds, max_processes
        self.isolation = strongest_isolation() if isolation == "auto" else isolation
        if self.isolation not in ("namespaces", "uid", "rlimits"):
            raise ValueError(f"unknown isolation {isolation!r}")
        if self.isolation == "namespaces" and namespace_command() is None:
            raise SandboxUnavailable("user / network / PID namespaces cannot be created on this host")
        if self.isolation == "uid" and os.geteuid() != 0:
            raise SandboxUnavailable("dropping to an unprivileged uid needs a root caller")
        if self.isolation == "rlimits" and not allow_unisolated:
            raise SandboxUnavailable("only resource limits are available here, which is not a security boundary; "
                                     "pass allow_unisolated=True to run trusted snippets anyway")
        self._dir = tempfile.TemporaryDirectory(prefix="archlab-sandbox-")
        self.root = Path(self._dir.name)
        self._drops_uid = os.geteuid() == 0 and self.isolation in ("namespaces", "uid")
        if self._drops_uid:
            os.chown(self.root, NOBODY, NOBODY)

    def _limits(self):
        resource.setrlimit(resource.RLIMIT_CPU, (self.cpu, self.cpu))
        resource.setrlimit(resource.RLIMIT_AS, (self.mem << 20, self.mem << 20))
        resource.setrlimit(resource.RLIMIT_NPROC, (self.nproc, self.nproc))

    def write(self, name: str, text: str) -> Path:
        p = (self.root / name).resolve()
        if self.root.resolve() not in p.parents:
            raise ValueError("path escapes the sandbox")
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(text)
        if self._drops_uid:
            os.chown(p, NOBODY, NOBODY)
        return p

    def _command(self, script: Path) -> tuple[list[str], dict]:
        inner = [sys.executable, "-I", str(script)]
        if self.isolation == "namespaces":
            return [*namespace_command(), *inner], {}
        if self.isolation == "uid":
            return inner, {"user": NOBODY, "group": NOBODY, "extra_groups": []}
        return inner, {}

    def run_python(self, code: str, *, stdin: str = "") -> ToolResult:
        script = self.write("_tool.py", code)
        cmd, ids = self._command(script)
        proc = subprocess.Popen(cmd, cwd=self.root, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                text=True, env={"PATH": os.environ.get("PATH", "")}, preexec_fn=self._limits,
                                start_new_session=True, **ids)
        try:
            out, err = proc.communicate(stdin, timeout=self.wall)
            timed_out = False
        except subprocess.TimeoutExpired:
            timed_out = True
            out, err = self._kill_group(proc)
        finally:
            self._signal_group(proc.pid)                          # descendants that outlived a normal exit
        return ToolResult(-9 if timed_out else proc.returncode, (out or "")[-8192:], (err or "")[-8192:], timed_out)

    @staticmethod
    def _signal_group(pgid: int) -> None:
        try:
            os.killpg(pgid, signal.SIGKILL)                       # session leader's pid == process group id
        except (ProcessLookupError, PermissionError):
            pass

    def _kill_group(self, proc) -> tuple[str, str]:
        self._signal_group(proc.pid)
        try:
            return proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:                         # a pipe held open elsewhere: give up on the output
            proc.kill()
            return "", ""

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


@dataclass(frozen=True)
class ExecutionResult:
    """Outcome of running one generated program (code-benchmark grading)."""
    success: bool
    stdout: str
    stderr: str
    error: str | None = None
    timeout: bool = False
    memory_exceeded: bool = False


def execute_code(code: str, *, timeout: float = 5.0, memory_mb: int = 256, allow_unisolated: bool = False) -> ExecutionResult:
    """Runs ``code`` (a complete program: solution plus its tests) in a fresh sandbox and classifies the outcome: success
    means exit code 0 within the time and memory limits.  A timeout kills the whole process group; an exhausted address
    space shows up as ``MemoryError`` and is reported as such rather than as a plain failure, so a grader can tell "wrong"
    from "too expensive".  The sandbox (and its directory) does not outlive the call.  Same role as the reference's
    generated-code executor (src/archlab/speedrun/execution.py:38-358), with the isolation described at the top of this
    module instead of in-process function patching."""
    isolation = strongest_isolation()
    with LocalSandbox(cpu_seconds=max(1, int(timeout) + 1), memory_mb=memory_mb, wall_seconds=timeout, isolation=isolation,
                      allow_unisolated=allow_unisolated or isolation != "rlimits") as box:
        r = box.run_python(code)
    if r.timed_out:
        return ExecutionResult(False, r.stdout, r.stderr, "execution timed out", timeout=True)
    if r.returncode == 0:
        return ExecutionResult(True, r.stdout, r.stderr)
    last = r.stderr.strip().splitlines()[-1] if r.stderr.strip() else f"exit code {r.returncode}"
    memory = "MemoryError" in r.stderr
    return ExecutionResult(False, r.stdout, r.stderr, "memory limit exceeded" if memory else last, memory_exceeded=memory)
