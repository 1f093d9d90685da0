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


def run_pytest(nodes, output, *, deployment=None, timeout: int = 1800, world_size: int = 1, env_extra=None,
               root: Path = ROOT) -> dict:
    """Run concrete pytest nodes of this checkout; a missing, failed or SKIPPED test never passes."""
    output = Path(output)
    output.mkdir(parents=True, exist_ok=True)
    for node in nodes:
        if not (root / node.split("::", 1)[0]).is_file():
            return dict(status="pending", reason="concrete integration test not implemented", node=node)
    report = output / "pytest.xml"
    reports = [output / f"pytest-rank-{r}.xml" for r in range(world_size)] if world_size > 1 else [report]
    for path in reports:
        path.unlink(missing_ok=True)
    cmd = [sys.executable]
    if world_size > 1:
        cmd += ["-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
                f"--nproc_per_node={world_size}"]
    cmd += ["-m", "pytest", "-q", *nodes, f"--basetemp={output.resolve() / 'artifacts'}", f"--junitxml={report}"]
    env = os.environ.copy()
    env.update(env_extra or {})
    if deployment is not None:
        for name in ("resolved.yaml", "experiment.json"):
            (output / name).write_bytes((Path(deployment) / name).read_bytes())
        env["ARCHLAB_QUALIFICATION_CONFIG"] = str((output / "resolved.yaml").resolve())
        env["ARCHLAB_QUALIFICATION_EXPERIMENT"] = str((output / "experiment.json").resolve())
        env.update(ARCHLAB_RUN_DISTRIBUTED="1", ARCHLAB_RUN_ENGINE="1", ARCHLAB_RUN_NATIVE_CONTEXT="1",
                   ARCHLAB_RUN_THROUGHPUT="1", ARCHLAB_RUN_AGENTIC_PIPELINE="1",
                   ARCHLAB_LEARNER_WORK=str(output / "learner"))
    env["ARCHLAB_JUNIT_PER_RANK"] = "1" if world_size > 1 else "0"
    sources = source_manifest(root)
    atomic_write_json(output / "source.json", sources)
    with (output / "pytest.log").open("w") as log:
        done = subprocess.run(cmd, cwd=root, env=env, stdout=log, stderr=subprocess.STDOUT, timeout=timeout)
    source = check_source_unchanged(sources, root)
    if not all(p.exists() for p in reports):
        raise RuntimeError(f"pytest did not produce a report (exit {done.returncode}); see {output / 'pytest.log'}")
    cases = [c for p in reports for c in ET.parse(p).iter("testcase")]
    if any(not list(ET.parse(p).iter("testcase")) for p in reports):
        raise RuntimeError(f"qualification tests failed or skipped: empty rank report; see {output / 'pytest.log'}")
    bad = [c.attrib.get("name") for c in cases
           if any(c.find(tag) is not None for tag in ("failure", "error", "skipped"))]
    if done.returncode or not cases or bad:
        raise RuntimeError(f"qualification tests failed or skipped: {bad}; see {output / 'pytest.log'}")
    return dict(status="passed", tests=len(cases), world_size=world_size, source=source,
                deployment_sha256=({n: sha256_file(output / n) for n in ("resolved.yaml", "experiment.json")}
                                   if deployment is not None else None),
                reports={str(p): sha256_file(p) for p in reports})


def check_learning_signal(output, pilot=None) -> dict:
    """A completed tool loop alone does not establish a useful policy update."""
    receipts = list((Path(output) / "artifacts").rglob("pipeline-evidence.json"))
    if len(receipts) != 1:
        raise ValueError("real policy update must write exactly one learning-signal receipt")
    ev = json.loads(receipts[0].read_text())
    contrast, grad_norm = ev["reward_contrast_groups"], ev["grad_norm"]
    if not isinstance(grad_norm, (int, float)) or not math.isfinite(grad_norm):
        raise ValueError("real policy update did not record a finite gradient norm")
    result = dict(receipt=str(receipts[0]), receipt_sha256=sha256_file(receipts[0]),
                  reward_contrast_groups=contrast, grad_norm=grad_norm)
    if pilot is None:
        if contrast <= 0 or grad_norm <= 0:
            result.update(status="pending", reason="execution passed but this pilot has no nonzero GRPO learning signal")
        return result
    obs = {k: ev.get(k, 0) for k in ("completed_verifiers", "tool_calls", "masked_observation_tokens",
                                     "truncated_trajectories")}
    obs["prompt_groups"] = len({uid.rsplit("_", 2)[0] for uid in ev.get("consumed_rollout_uids", [])})
    obs["reward_contrast_groups"] = contrast
    limits = dict(completed_verifiers=pilot.minimum_completed_verifiers, prompt_groups=pilot.minimum_prompt_groups,
                  tool_calls=pilot.minimum_tool_calls, masked_observation_tokens=pilot.minimum_observation_tokens,
                  reward_contrast_groups=pilot.minimum_reward_contrast_groups)
    failed = [k for k, lo in limits.items() if type(obs[k]) is not int or obs[k] < lo]
    if type(obs["truncated_trajectories"]) is not int or obs["truncated_trajectories"] > pilot.maximum_truncated_trajectories:
        failed.append("truncated_trajectories")
    if grad_norm <= 0:
        failed.append("positive_gradient")
    result.update(observed=obs, thresholds=asdict(pilot))
    if failed:
        result.update(status="failed", reason="bootstrap pilot health thresholds not met: " + ", ".join(failed))
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
