"""Speedrun entry on CPU: lifecycle flags (budget guards, declared initialisation hash, metrics and checkpoint
locations, throughput summary, final-checkpoint switch)."""
import json

import pytest

from archlab_b200.train import base_train

ARGS = ["--depth=2", "--max-seq-len=32", "--vocab-size=256", "--device-batch-size=2", "--total-batch-size=128",
        "--num-iterations=4", "--throughput-warmup-steps=1"]


@pytest.fixture(autouse=True)
def _single_process(monkeypatch):
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)


def test_run_writes_metrics_checkpoint_and_throughput(tmp_path):
    ck, mp = tmp_path / "ck", tmp_path / "m.jsonl"
    assert base_train.main(ARGS + [f"--run-dir={tmp_path / 'run'}", f"--checkpoint-dir={ck}", f"--metrics-path={mp}",
                                   "--metrics-every=2"]) == 0
    rows = [json.loads(l) for l in open(mp)]
    assert [r["step"] for r in rows] == [2, 4]
    assert any(p.name.startswith("model_000004") for p in ck.iterdir())
    thr = json.loads((tmp_path / "run" / "throughput.json").read_text())
    assert thr["throughput_protocol"]["warmup_steps"] == 1 and thr["throughput_sample_intervals"] >= 1
    assert thr["steady_state_tokens_per_second"] > 0


def test_budget_guards_and_initialisation_hash(tmp_path):
    with pytest.raises(SystemExit, match="max-parameters"):
        base_train.main(ARGS + [f"--run-dir={tmp_path}", "--max-parameters=10"])
    with pytest.raises(SystemExit, match="max-training-tokens"):
        base_train.main(ARGS + [f"--run-dir={tmp_path}", "--max-training-tokens=256"])
    with pytest.raises(SystemExit, match="initial weights"):
        base_train.main(ARGS + [f"--run-dir={tmp_path}", "--initialization-hash=00"])


def test_final_checkpoint_can_be_switched_off(tmp_path):
    assert base_train.main(ARGS + [f"--run-dir={tmp_path}", "--no-final-checkpoint"]) == 0
    assert not (tmp_path / "checkpoints").exists() or not list((tmp_path / "checkpoints").iterdir())
