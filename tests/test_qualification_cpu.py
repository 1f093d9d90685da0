"""Admission gates on CPU: a pytest gate passes only on all-passed reports, and the learning-signal receipt check."""
import json
from pathlib import Path

import pytest

from archlab_b200.contracts.experiment import AgenticPilot
from archlab_b200.train import qualification as q


def _checkout(tmp_path: Path, body: str) -> Path:
    root = tmp_path / "checkout"
    (root / "tests").mkdir(parents=True)
    (root / "tests" / "test_gate.py").write_text(body)
    return root


def test_gate_passes_only_when_every_case_passed(tmp_path):
    root = _checkout(tmp_path, "def test_ok():\n    assert True\n")
    out = q.run_pytest(["tests/test_gate.py::test_ok"], tmp_path / "out", root=root)
    assert out["status"] == "passed" and out["tests"] == 1 and out["world_size"] == 1 and out["deployment_sha256"] is None
    assert len(out["reports"]) == 1 and (tmp_path / "out" / "pytest.log").is_file()


@pytest.mark.parametrize("body", ["def test_ok():\n    assert False\n",
                                  "import pytest\n\ndef test_ok():\n    pytest.skip('no accelerator')\n"])
def test_failed_or_skipped_case_is_refused(tmp_path, body):
    root = _checkout(tmp_path, body)
    with pytest.raises(RuntimeError, match="failed or skipped"):
        q.run_pytest(["tests/test_gate.py"], tmp_path / "out", root=root)


def test_missing_node_is_pending_and_deployment_is_frozen(tmp_path):
    root = _checkout(tmp_path, "import os\n\ndef test_env():\n    assert os.environ['ARCHLAB_RUN_ENGINE'] == '1'\n"
                               "    assert open(os.environ['ARCHLAB_QUALIFICATION_CONFIG']).read() == 'a: 1\\n'\n")
    pending = q.run_pytest(["tests/test_absent.py::test_x"], tmp_path / "p", root=root)
    assert pending["status"] == "pending" and pending["node"].startswith("tests/test_absent.py")
    deployment = tmp_path / "deployment"
    deployment.mkdir()
    (deployment / "resolved.yaml").write_text("a: 1\n")
    (deployment / "experiment.json").write_text("{}")
    out = q.run_pytest(["tests/test_gate.py"], tmp_path / "out", deployment=deployment, root=root)
    assert set(out["deployment_sha256"]) == {"resolved.yaml", "experiment.json"}


def test_source_change_during_a_gate_is_refused(tmp_path):
    root = _checkout(tmp_path, "from pathlib import Path\n\ndef test_edit():\n"
                               "    Path(__file__).with_name('test_new.py').write_text('x = 1\\n')\n")
    with pytest.raises(RuntimeError, match="source changed"):
        q.run_pytest(["tests/test_gate.py"], tmp_path / "out", root=root)


def _receipt(out: Path, **fields):
    d = out / "artifacts" / "run"
    d.mkdir(parents=True, exist_ok=True)
    base = {"reward_contrast_groups": 2, "grad_norm": 0.5, "completed_verifiers": 8, "tool_calls": 3, "masked_observation_tokens": 40,
            "truncated_trajectories": 0, "consumed_rollout_uids": [f"p{g}_{i}_0" for g in range(2) for i in range(4)]}
    (d / "pipeline-evidence.json").write_text(json.dumps({**base, **fields}))


def test_learning_signal_receipt(tmp_path):
    with pytest.raises(ValueError, match="exactly one"):
        q.check_learning_signal(tmp_path)
    _receipt(tmp_path)
    ok = q.check_learning_signal(tmp_path, AgenticPilot())
    assert "status" not in ok and ok["observed"]["prompt_groups"] == 2
    _receipt(tmp_path, tool_calls=0, truncated_trajectories=1)
    bad = q.check_learning_signal(tmp_path, AgenticPilot())
    assert bad["status"] == "failed" and "tool_calls" in bad["reason"] and "truncated_trajectories" in bad["reason"]
    _receipt(tmp_path, reward_contrast_groups=0)
    assert q.check_learning_signal(tmp_path)["status"] == "pending"
    _receipt(tmp_path, grad_norm=float("nan"))
    with pytest.raises(ValueError, match="finite"):
        q.check_learning_signal(tmp_path)
