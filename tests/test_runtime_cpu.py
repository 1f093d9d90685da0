"""Launch plans, the speedrun entry (CPU, 1 process) and checkpoint resume."""
import json
import sys
from types import SimpleNamespace

import pytest
import torch

from archlab_b200.train import backends, runtime


def test_speedrun_plan_is_inspectable():
    plan = backends.SpeedrunBackend().render(depth=20, topology=backends.Topology(gpus_per_node=8))
    assert plan.metadata["grad_accum_steps"] == 2 and plan.metadata["world_size"] == 8
    sh = plan.shell()
    assert "archlab_b200.train.base_train" in sh and '"${ARCHLAB_RUN_DIR}"' in sh and "--nproc-per-node=8" in sh
    with pytest.raises(ValueError):
        backends.SpeedrunBackend().render(total_batch_size=1000)


def test_mesh_plan_validates_parallel_sizes():
    plan = backends.MeshBackend().render(model="qwen35_4b", tp=2, global_batch=128, topology=backends.Topology())
    assert plan.metadata["data_parallel"] == 4 and "tp2+sp" in plan.metadata["parallelism"]
    assert "--sequence-parallel" in plan.argv
    with pytest.raises(ValueError):
        backends.MeshBackend().render(model="m", tp=3)
    with pytest.raises(ValueError):
        backends.MeshBackend().render(model="m", ep=3)
    with pytest.raises(ValueError):
        backends.MeshBackend().render(model="m", precision="int3")


def test_runtime_dry_run_writes_plan(tmp_path):
    exp = SimpleNamespace(engine="speedrun", family="nanochat", settings={"depth": 4, "total_batch_size": 16 * 2048})
    assert runtime.run(exp, {}, tmp_path, gpus=1, dry_run=True) == 0
    plan = json.loads((tmp_path / "launch_plan.json").read_text())
    assert plan["backend"] == "speedrun" and "--depth=4" in plan["argv"]
    assert (tmp_path / "launch.sh").read_text().startswith("#!/bin/sh")


def test_worker_environment_keeps_tracking_private(tmp_path):
    cfg = tmp_path / "tracking.json"
    cfg.write_text(json.dumps({"tracking_uri": "http://127.0.0.1:1", "token": "s3cret"}))
    env = runtime.worker_environment({"ARCHLAB_MLFLOW_CONFIG": str(cfg)})
    assert env["MLFLOW_TRACKING_TOKEN"] == "s3cret"


@pytest.mark.slow
def test_base_train_runs_and_resumes_on_cpu(tmp_path):
    from archlab_b200.train import base_train

    common = ["--depth", "2", "--max-seq-len", "32", "--vocab-size", "256", "--device-batch-size", "2",
              "--total-batch-size", "64", "--run-dir", str(tmp_path), "--warmup-steps", "1"]
    assert base_train.main(common + ["--num-iterations", "3", "--save-every", "2"]) == 0
    lines = [json.loads(l) for l in (tmp_path / "metrics_rank0.jsonl").read_text().splitlines()]
    assert [l["step"] for l in lines] == [1, 2, 3] and all(torch.isfinite(torch.tensor(l["loss"])) for l in lines)
    assert (tmp_path / "checkpoints" / "model_000002.pt").is_file()
    assert base_train.main(common + ["--num-iterations", "4", "--resume-from-step", "2"]) == 0
    lines = [json.loads(l) for l in (tmp_path / "metrics_rank0.jsonl").read_text().splitlines()]
    assert [l["step"] for l in lines][-2:] == [3, 4]
