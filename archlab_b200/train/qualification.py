"""Fail-closed admission report for one resolved deployment.

The structure follows the reference's ``qualify`` (src/archlab/training/qualification.py:538-629):
an ordered list of checks, each reduced to ``passed`` / ``failed`` / ``pending``; readiness checks
(configuration science, source identity, runtime, data, model lineage, native fixtures) gate the
GPU integration gates, which run this checkout's own pytest nodes in a subprocess (one process per
GPU through ``torch.distributed.run`` when a gate is distributed); a skipped test is a failure;
prerequisites are explicit; the source tree is fingerprinted before and after.  The result is
``qualification.json`` and ``result["passed"]`` gates ``archlab train``.
"""
from __future__ import annotations

import hashlib
import importlib
import importlib.metadata
import json
import math
import os
import subprocess
import sys
import time
import xml.etree.ElementTree as ET
from dataclasses import asdict
from pathlib import Path

import yaml

from ..contracts.experiment import Experiment, fingerprint, validate_science
from ..contracts.performance import check_throughput
from ..contracts.substrate import atomic_write_json, sha256_file

ROOT = Path(__file__).resolve().parents[2]
FORMAT = "archlab-training-qualification-v1"

# gate -> (pytest node under tests/integration, runs one process per GPU?)
INTEGRATION_TESTS = {
    "native_distributed_oracle": ("test_learner_gates.py::test_native_forward_backward", True),
    "package_optimizer_restart": ("test_learner_gates.py::test_optimizer_checkpoint_restart", True),
    "serving_reload_parity": ("test_serving_gates.py::test_full_checkpoint_short_context_parity", False),
    "native_context_backward": ("test_learner_gates.py::test_native_context_forward_backward_memory", False),
    "native_context_serving": ("test_serving_gates.py::test_native_context_capacity", False),
    "learner_throughput": ("test_learner_gates.py::test_package_learner_throughput", True),
    "agent_tool_verifier": ("test_sandbox_gates.py::test_agent_tool_and_successful_verifier", False),
    "real_policy_grpo_update": ("test_pipeline_gates.py::test_real_policy_grpo_update", False),
}
PREREQUISITES = {
    "serving_reload_parity": ("package_optimizer_restart",),
    "agent_tool_verifier": ("sandbox_coverage",),
    "real_policy_grpo_update": ("native_distributed_oracle", "package_optimizer_restart", "serving_reload_parity",
                                "native_context_backward", "native_context_serving", "throughput_regression",
                                "sandbox_coverage", "agent_tool_verifier"),
}
SPEEDRUN_TESTS = {
    "kernel_numerics": ("tests/test_gemm_gpu.py", False),
    "engine_gradient_oracle": ("tests/test_engine_gpu.py", False),
}


# ------------------------------------------------------------------------------------------------
def source_manifest(root: Path = ROOT) -> dict[str, str]:
    """sha256 of the actual source bytes, committed or not."""
    files = set()
    for directory in ("archlab_b200", "tests", "recipes"):
        base = root / directory
        if base.is_dir():
            files.update(p for p in base.rglob("*") if p.is_file()
                         and p.suffix in {".py", ".yaml", ".yml", ".cu", ".cuh", ".h"} and "build" not in p.parts)
    files.update(root / n for n in ("bench.py", "__graft_entry__.py") if (root / n).is_file())
    return {str(p.relative_to(root)): sha256_file(p) for p in sorted(files)}


def check_source_unchanged(expected: dict[str, str], root: Path = ROOT) -> dict:
    actual = source_manifest(root)
    changed = sorted(n for n in expected.keys() | actual.keys() if expected.get(n) != actual.get(n))
    if changed:
        raise RuntimeError("source changed during admission: " + ", ".join(changed[:10]))
    return {"files": len(actual), "sha256": hashlib.sha256(json.dumps(actual, sort_keys=True).encode()).hexdigest()}


def check_runtime(experiment: Experiment, config: dict) -> dict:
    """Interpreter, packages, native library and visible accelerators of THIS deployment."""
    import torch

    pkgs = {}
    for name in ("torch", "numpy", "pyyaml", "safetensors"):
        try:
            pkgs[name] = importlib.metadata.version(name)
        except importlib.metadata.PackageNotFoundError as e:
            raise ValueError(f"required package missing: {name}") from e
    if sys.version_info < (3, 10):
        raise ValueError("Python >= 3.10 is required")
    want = int(config["trainer"]["nnodes"]) * int(config["trainer"]["n_gpus_per_node"])
    have = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if experiment.family != "speedrun" and have < int(config["trainer"]["n_gpus_per_node"]):
        raise ValueError(f"deployment needs {want} GPUs, this host exposes {have}")
    lib = ROOT / "archlab_b200" / "libnga_b200.so"
    if have and not lib.is_file():
        raise ValueError("native library is not built")
    names = sorted({torch.cuda.get_device_name(i) for i in range(have)})
    return {"python": sys.version.split()[0], "packages": pkgs, "gpus": have, "gpu_names": names,
            "native_library_sha256": sha256_file(lib) if lib.is_file() else None}


def check_data(experiment: Experiment, config: dict, output: Path) -> dict:
    manifest = Path(experiment.data_manifest)
    if not manifest.is_file():
        raise FileNotFoundError(f"data manifest not found: {manifest}")
    body = json.loads(manifest.read_text())
    files = body.get("files", [])
    if not files:
        raise ValueError("data manifest lists no files")
    missing = [f["path"] for f in files if not (manifest.parent / f["path"]).is_file()]
    if missing:
        raise ValueError("data manifest members are missing: " + ", ".join(missing[:5]))
    return {"manifest": str(manifest), "manifest_sha256": sha256_file(manifest), "files": len(files)}


def check_model(experiment: Experiment, config: dict) -> dict:
    ckpt = Path(experiment.parent_checkpoint)
    if not ckpt.exists():
        raise FileNotFoundError(f"parent checkpoint not found: {ckpt}")
    export = ckpt / "EXPORT.json"
    detail = {"parent_checkpoint": str(ckpt), "parent_stage": experiment.parent_stage}
    if export.is_file():
        meta = json.loads(export.read_text())
        for name, digest in meta.get("files", {}).items():
            if sha256_file(ckpt / name) != digest:
                raise ValueError(f"export member differs from its recorded hash: {name}")
        detail["export_format"] = meta.get("format")
        detail["state_sha256"] = meta.get("state_sha256")
    return detail


GATE_SWITCHES = ("DISTRIBUTED", "ENGINE", "NATIVE_CONTEXT", "THROUGHPUT", "AGENTIC_PIPELINE")   # ARCHLAB_RUN_<switch>=1
DEPLOYMENT_FILES = {"resolved.yaml": "ARCHLAB_QUALIFICATION_CONFIG", "experiment.json": "ARCHLAB_QUALIFICATION_EXPERIMENT"}
_NOT_A_PASS = ("failure", "error", "skipped")


class _PytestGate:
    """One subprocess run of pytest nodes of this checkout, one process per GPU when ``world_size`` > 1.

    Every rank writes its own junit report (the test session reads ``ARCHLAB_JUNIT_PER_RANK``); a gate passes only when
    every report exists, holds at least one test case, and no case failed, errored or was skipped."""

    def __init__(self, nodes, output: Path, world_size: int, root: Path):
        self.nodes, self.output, self.world, self.root = list(nodes), output, world_size, root
        self.reports = [output / f"pytest-rank-{r}.xml" for r in range(world_size)] if world_size > 1 else [output / "pytest.xml"]

    def unimplemented(self):
        return next((n for n in self.nodes if not (self.root / n.partition("::")[0]).is_file()), None)

    def command(self) -> list[str]:
        launcher = ["-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
                    f"--nproc_per_node={self.world}"] if self.world > 1 else []
        return [sys.executable, *launcher, "-m", "pytest", "-q", *self.nodes,
                f"--basetemp={self.output.resolve() / 'artifacts'}", f"--junitxml={self.output / 'pytest.xml'}"]

    def environment(self, deployment, extra) -> dict:
        env = {**os.environ, **(extra or {}), "ARCHLAB_JUNIT_PER_RANK": str(int(self.world > 1))}
        if deployment is not None:                       # the gate reads the frozen copy, not the caller's files
            for name, variable in DEPLOYMENT_FILES.items():
                (self.output / name).write_bytes((Path(deployment) / name).read_bytes())
                env[variable] = str((self.output / name).resolve())
            env.update({f"ARCHLAB_RUN_{switch}": "1" for switch in GATE_SWITCHES})
            env["ARCHLAB_LEARNER_WORK"] = str(self.output / "learner")
        return env

    def verdict(self, exit_code: int) -> int:
        log = self.output / "pytest.log"
        if absent := [p.name for p in self.reports if not p.exists()]:
            raise RuntimeError(f"pytest did not produce a report (exit {exit_code}; missing {absent}); see {log}")
        per_rank = [list(ET.parse(p).iter("testcase")) for p in self.reports]
        if not all(per_rank):
            raise RuntimeError(f"qualification tests failed or skipped: empty rank report; see {log}")
        not_passed = [case.get("name") for cases in per_rank for case in cases if any(case.find(t) is not None for t in _NOT_A_PASS)]
        if exit_code or not_passed:
            raise RuntimeError(f"qualification tests failed or skipped: {not_passed}; see {log}")
        return sum(map(len, per_rank))


def run_pytest(nodes, output, *, deployment=None, timeout: int = 1800, world_size: int = 1, env_extra=None,
               root: Path = ROOT) -> dict:
    """Run concrete pytest nodes of this checkout; a missing, failed or SKIPPED test never passes."""
    output = Path(output)
    output.mkdir(parents=True, exist_ok=True)
    gate = _PytestGate(nodes, output, world_size, root)
    if (node := gate.unimplemented()) is not None:
        return dict(status="pending", reason="concrete integration test not implemented", node=node)
    for stale in gate.reports:
        stale.unlink(missing_ok=True)
    env = gate.environment(deployment, env_extra)
    before = source_manifest(root)
    atomic_write_json(output / "source.json", before)
    with (output / "pytest.log").open("w") as log:
        exit_code = subprocess.run(gate.command(), cwd=root, env=env, stdout=log, stderr=subprocess.STDOUT, timeout=timeout).returncode
    source = check_source_unchanged(before, root)
    tests = gate.verdict(exit_code)
    frozen = {n: sha256_file(output / n) for n in DEPLOYMENT_FILES} if deployment is not None else None
    return dict(status="passed", tests=tests, world_size=world_size, source=source, deployment_sha256=frozen,
                reports={str(p): sha256_file(p) for p in gate.reports})


# pilot threshold field -> observed counter it bounds from below
PILOT_FLOORS = {"minimum_completed_verifiers": "completed_verifiers", "minimum_prompt_groups": "prompt_groups",
                "minimum_tool_calls": "tool_calls", "minimum_observation_tokens": "masked_observation_tokens",
                "minimum_reward_contrast_groups": "reward_contrast_groups"}


def check_learning_signal(output, pilot=None) -> dict:
    """A completed tool loop alone does not establish a useful policy update: the update's receipt must show a finite,
    positive gradient norm and reward contrast, and - with pilot thresholds - enough verifiers, groups, tool calls and
    observation tokens and few enough truncations."""
    found = list((Path(output) / "artifacts").rglob("pipeline-evidence.json"))
    if len(found) != 1:
        raise ValueError("real policy update must write exactly one learning-signal receipt")
    evidence = json.loads(found[0].read_text())
    contrast, grad_norm = evidence["reward_contrast_groups"], evidence["grad_norm"]
    if not isinstance(grad_norm, (int, float)) or not math.isfinite(grad_norm):
        raise ValueError("real policy update did not record a finite gradient norm")
    result = dict(receipt=str(found[0]), receipt_sha256=sha256_file(found[0]), reward_contrast_groups=contrast, grad_norm=grad_norm)
    if pilot is None:
        if min(contrast, grad_norm) <= 0:
            result.update(status="pending", reason="execution passed but this pilot has no nonzero GRPO learning signal")
        return result
    groups = {uid.rsplit("_", 2)[0] for uid in evidence.get("consumed_rollout_uids", [])}
    observed = {counter: evidence.get(counter, 0) for counter in (*PILOT_FLOORS.values(), "truncated_trajectories")}
    observed.update(prompt_groups=len(groups), reward_contrast_groups=contrast)
    whole = lambda v: type(v) is int
    short = [counter for floor, counter in PILOT_FLOORS.items() if not whole(observed[counter]) or observed[counter] < getattr(pilot, floor)]
    if not whole(observed["truncated_trajectories"]) or observed["truncated_trajectories"] > pilot.maximum_truncated_trajectories:
        short.append("truncated_trajectories")
    if grad_norm <= 0:
        short.append("positive_gradient")
    result.update(observed=observed, thresholds=asdict(pilot))
    if short:
        result.update(status="failed", reason="bootstrap pilot health thresholds not met: " + ", ".join(short))
    return result


def _check(name: str, fn) -> dict:
    t0 = time.monotonic()
    try:
        detail = fn() or {}
        row = dict(name=name, **{"status": "passed", **detail})
    except Exception as e:  # every failure becomes a recorded blocker
        row = dict(name=name, status="failed", reason=f"{type(e).__name__}: {e}")
    row["seconds"] = time.monotonic() - t0
    return row


def qualify(experiment: Experiment, config: dict, output, *, run_gates: bool = True) -> dict:
    output = Path(output)
    output.mkdir(parents=True, exist_ok=True)
    (output / "resolved.yaml").write_text(yaml.safe_dump(config, sort_keys=False))
    atomic_write_json(output / "experiment.json", asdict(experiment))
    sources = source_manifest()
    atomic_write_json(output / "source.json", sources)
    speedrun = experiment.family == "speedrun"
    checks = [_check("scientific_config", (lambda: {}) if speedrun else (lambda: validate_science(experiment, config))),
              _check("deployment_runtime", lambda: check_runtime(experiment, config))]
    if not speedrun:
        checks += [_check("agentic_data", lambda: check_data(experiment, config, output)),
                   _check("model_export", lambda: check_model(experiment, config))]
    checks.append(_check("native_model_fixture", lambda: run_pytest(
        ["tests/test_contracts.py"], output / "native_fixture", deployment=None)))
    if run_gates and "simplicial" in json.dumps(asdict(experiment), default=str).lower():
        # kernel preflight before anything trains with the 2-simplicial op: FP64 ladder + causality (+ timing on a GPU)
        from .preflight_simplicial import run as simplicial_preflight

        def preflight():
            receipt = output / "simplicial_preflight.json"
            receipt.unlink(missing_ok=True)
            ev = simplicial_preflight(receipt, repetitions=5)
            return {"receipt": receipt.name, "cases": len(ev["correctness"]), "benchmarks": len(ev["benchmarks"])}

        checks.append(_check("simplicial_kernel_preflight", preflight))
    ready = all(r["status"] == "passed" for r in checks)
    if speedrun:
        plan = {k: (v[0], v[1]) for k, v in SPEEDRUN_TESTS.items()}
    else:
        plan = {k: (f"tests/integration/{v[0]}", v[1]) for k, v in INTEGRATION_TESTS.items()}
        checks.append(_check("sandbox_coverage", lambda: _sandbox_coverage(experiment, config)))
    for test, (node, distributed) in plan.items():
        if not (ready and run_gates):
            checks.append(dict(name=test, status="pending", reason="deployment readiness checks failed"
                               if not ready else "integration gates were not requested"))
            continue
        passed = {r["name"] for r in checks if r["status"] == "passed"}
        missing = sorted(set(PREREQUISITES.get(test, ())) - passed)
        if missing:
            checks.append(dict(name=test, status="pending", reason="prerequisites not passed: " + ", ".join(missing)))
            continue
        ws = int(config["trainer"]["n_gpus_per_node"]) if distributed else 1
        checks.append(_check(test, lambda node=node, test=test, ws=ws: run_pytest(
            [node], output / test, deployment=output, world_size=ws,
            timeout=14760 if test == "real_policy_grpo_update" else 1800)))
        if test == "learner_throughput":
            if checks[-1]["status"] == "passed":
                checks.append(_check("throughput_regression", lambda test=test: check_throughput(
                    experiment.throughput, output / test / "throughput.json")))
            else:
                checks.append(dict(name="throughput_regression", status="pending",
                                   reason="learner benchmark has not passed"))
    if not speedrun:
        if any(r["name"] == "real_policy_grpo_update" and r["status"] == "passed" for r in checks):
            checks.append(_check("agentic_learning_signal", lambda: check_learning_signal(
                output / "real_policy_grpo_update", experiment.pilot)))
        else:
            checks.append(dict(name="agentic_learning_signal", status="pending",
                               reason="real policy update has not passed"))
    checks.append(_check("source_unchanged", lambda: check_source_unchanged(sources)))
    result = dict(format=FORMAT, passed=all(r["status"] == "passed" for r in checks),
                  config_sha256=fingerprint(config), checks=checks,
                  blockers=[r["name"] for r in checks if r["status"] != "passed"])
    atomic_write_json(output / "qualification.json", result)
    return result


def _sandbox_coverage(experiment: Experiment, config: dict) -> dict:
    from .sandbox import check_sandbox

    return check_sandbox(experiment, config)
