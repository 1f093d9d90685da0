"""A fail-closed sequential campaign over the arms of a comparison (A / B / C): every arm trains only after ALL arms'
probes proved that they would see the same run, and a later arm never starts on changed sources.

``validate_probes`` reads, per arm, the probe's evidence: ``PROBE_COMPLETE.json`` (weights, scheduler and optimizer were
restored bit for bit from the probe checkpoint), ``RUN_CONTRACT.json`` (must name this arm, mode "probe", the same
runtime / topology / seed / batch / data manifest / held-out set as the other arms, and source hashes equal to the
sources about to be launched), ``INITIALIZATION.json`` (the parameters all arms share start from the same digest) and
``metrics.jsonl`` (the same first micro-batches in the same order, the same held-out windows).

``ArmCampaign.run`` is fresh-only (an existing ``CAMPAIGN.json`` needs a person's review), takes a host-local advisory
lock, launches one child per arm in its own session, and on SIGTERM / SIGINT asks the ACTIVE arm to stop at its next
complete optimizer step by writing ``STOP_REQUESTED.json`` into its run directory (no signal is sent to the trainer, so
its launcher's short kill timeout never cuts a checkpoint).  An arm counts as complete only with exit code 0 and a
``TRAINING_COMPLETE.json`` whose consumed tokens equal the campaign's budget; anything else ends the campaign.
(Reference: src/archlab/megatron/simplicial_campaign.py:23-167.)
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import signal
import subprocess
import time
from pathlib import Path
from typing import Callable

from ..contracts.substrate import atomic_write_json

MATCHED = ("runtime", "topology", "seed", "global_batch", "micro_batch", "manifest_sha256", "train_prefixes", "heldout_prefixes", "eval_sequences")
RESTORED = ("all_model_weights_bitwise_restored", "scheduler_restored", "optimizer_tensors_bitwise_restored")


def source_hashes(root) -> dict[str, str]:
    root = Path(root)
    return {str(p.relative_to(root)): hashlib.sha256(p.read_bytes()).hexdigest() for p in sorted(root.rglob("*.py"))}


def _json(path: Path):
    return json.loads(path.read_text())


def validate_probes(probes: dict[str, Path], sources: dict[str, str], *, probe_steps: int = 3) -> dict:
    shared = init = order = heldout = None
    for arm, probe in probes.items():
        probe = Path(probe)
        done = _json(probe / "PROBE_COMPLETE.json")
        if not all(done.get(k) is True for k in RESTORED):
            raise ValueError(f"{arm}: checkpoint / optimizer restoration gate incomplete")
        contract = _json(probe / "RUN_CONTRACT.json")
        if contract["arm"] != arm or contract["mode"] != "probe":
            raise ValueError(f"{arm}: wrong probe evidence")
        matched = {k: contract[k] for k in MATCHED}
        if shared is not None and matched != shared:
            raise ValueError("probe runtime / data / batch contracts differ between arms")
        shared = matched
        if any(sources.get(name) != digest for name, digest in contract["source_sha256"].items()):
            raise ValueError(f"{arm}: the probe did not validate these exact sources")
        digest = _json(probe / "INITIALIZATION.json")["common_parameter_sha256"]
        if init is not None and digest != init:
            raise ValueError("probe initialisation mismatch")
        init = digest
        rows = [json.loads(line) for line in (probe / "metrics.jsonl").read_text().splitlines() if line.strip()]
        batches = [r["first_microbatches_sha256"] for r in rows if r["event"] == "train"]
        if len(batches) != probe_steps or (order is not None and batches != order):
            raise ValueError("probe data-order mismatch")
        order = batches
        windows = {r["heldout_tokens_sha256"] for r in rows if r["event"] == "eval"}
        if len(windows) != 1 or (heldout is not None and windows != heldout):
            raise ValueError("probe held-out window mismatch")
        heldout = windows
    return {"contract": shared, "common_parameter_sha256": init, "data_order": order, "heldout": sorted(heldout)}


class ArmCampaign:
    def __init__(self, root, source_root, command_for_arm: Callable[[str, Path], list[str]], *, expected_tokens: int, source_commit: str = "",
                 lock_path=None, poll_seconds: float = 1.0):
        self.root, self.source_root, self.command_for_arm = Path(root).resolve(), Path(source_root), command_for_arm
        self.expected_tokens, self.source_commit, self.poll = expected_tokens, source_commit, poll_seconds
        self.lock_path = Path(lock_path) if lock_path else self.root.parent / f".{self.root.name}.lock"
        self._stop, self._active = False, None

    def request_stop(self, *_):
        self._stop = True
        if self._active is not None and self._active.is_dir():
            atomic_write_json(self._active / "STOP_REQUESTED.json", {"requested_unix": time.time()})

    def run(self, probes: dict[str, Path], *, install_signal_handlers: bool = True) -> dict:
        self.root.mkdir(parents=True, exist_ok=True)
        state_path = self.root / "CAMPAIGN.json"
        if state_path.exists():
            raise ValueError("a campaign is fresh-only; resuming one needs explicit review")
        with self.lock_path.open("a") as lock:
            try:
                fcntl.flock(lock.fileno(), fcntl.LOCK_EX | fcntl.LOCK_NB)
            except BlockingIOError as busy:
                raise RuntimeError("another campaign holds this host's lock") from busy
            try:
                return self._run(probes, state_path, install_signal_handlers)
            except Exception as error:
                atomic_write_json(self.root / "FAILURE.json", {"error": repr(error), "time_unix": time.time()})
                if state_path.exists():
                    atomic_write_json(state_path, {**_json(state_path), "status": "failed", "error": repr(error)})
                raise

    def _run(self, probes, state_path, install_signal_handlers) -> dict:
        sources = source_hashes(self.source_root)
        evidence = validate_probes(probes, sources)
        arms = list(probes)
        state = {"source_commit": self.source_commit, "source_sha256": sources, "started_unix": time.time(), "supervisor_pid": os.getpid(),
                 "arms": {a: "queued" for a in arms}, "status": "running", "probe_evidence": evidence}
        atomic_write_json(state_path, state)
        if install_signal_handlers:
            signal.signal(signal.SIGTERM, self.request_stop)
            signal.signal(signal.SIGINT, self.request_stop)
        for arm in arms:
            if self._stop:
                break
            if source_hashes(self.source_root) != sources:
                raise RuntimeError("the source snapshot changed; refusing to launch the next arm")
            run_dir = self.root / arm
            self._active = run_dir
            with (self.root / f"{arm}.log").open("x") as log:
                child = subprocess.Popen(self.command_for_arm(arm, run_dir), stdin=subprocess.DEVNULL, stdout=log, stderr=subprocess.STDOUT,
                                         start_new_session=True)
                state.update(active_arm=arm, child_pid=child.pid)
                state["arms"][arm] = "running"
                atomic_write_json(state_path, state)
                while child.poll() is None:
                    if self._stop and run_dir.is_dir() and not (run_dir / "STOP_REQUESTED.json").exists():
                        atomic_write_json(run_dir / "STOP_REQUESTED.json", {"requested_unix": time.time()})
                    time.sleep(self.poll)
            done = run_dir / "TRAINING_COMPLETE.json"
            if child.returncode != 0 or not done.is_file():
                state["arms"][arm] = "stopped" if self._stop else "failed"
                state.update(status=state["arms"][arm], exit_code=child.returncode)
                atomic_write_json(state_path, state)
                return state
            if _json(done).get("consumed_tokens") != self.expected_tokens:
                raise RuntimeError(f"{arm}: incorrect completion token count")
            state["arms"][arm] = "complete"
            atomic_write_json(state_path, state)
        state.update(status="stopped" if self._stop else "complete", finished_unix=time.time())
        atomic_write_json(state_path, state)
        return state
