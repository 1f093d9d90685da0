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


def test_eval_cadence_validation_core_and_samples(tmp_path):
    tasks = {"parity": {"random_baseline": 0.5, "items": [{"prefix": [1, 2, 3], "choices": [[4, 5], [6]], "gold": 0},
                                                         {"prefix": [7], "choices": [[8], [9, 10]], "gold": 1}]}}
    (tmp_path / "tasks.json").write_text(json.dumps(tasks))
    (tmp_path / "prompts.yaml").write_text("prompts:\n  - [1, 2, 3]\n  - [9]\n")
    mp = tmp_path / "m.jsonl"
    assert base_train.main(ARGS + [f"--run-dir={tmp_path / 'run'}", f"--metrics-path={mp}", "--eval-every=2", "--eval-tokens=256",
                                   "--core-metric-every=2", f"--core-tasks={tmp_path / 'tasks.json'}", "--sample-every=4",
                                   f"--prompt-file={tmp_path / 'prompts.yaml'}", "--exact-global-batch-replay",
                                   "--no-final-checkpoint"]) == 0
    rows = [json.loads(l) for l in open(mp)]
    val = [r for r in rows if r["kind"] == "validation"]
    assert [r["step"] for r in val] == [0, 2, 4] and all(r["bpb"] > 0 and r["eval_tokens"] == 256 for r in val)
    assert val[-1]["total_training_flops"] > val[1]["total_training_flops"] > 0
    core = [r for r in rows if r["kind"] == "core"]
    assert [r["step"] for r in core] == [2, 4] and -1.0 <= core[0]["core_metric"] <= 1.0 and set(core[0]["centered_results"]) == {"parity"}
    samples = [r for r in rows if r["kind"] == "samples"]
    assert [r["step"] for r in samples] == [4] and [len(s) for s in samples[0]["samples"]] == [16, 16]
    train = [r for r in rows if r["kind"] == "train"]
    assert [r["step"] for r in train] == [1, 2, 3, 4] and train[-1]["smooth_loss"] > 0


def test_flop_budget_sets_the_horizon_and_loop_state_resumes(tmp_path):
    run = tmp_path / "run"
    base = [a for a in ARGS if not a.startswith("--num-iterations")]
    probe = base_train.parse_args(base)
    from archlab_b200.models.nanochat import GPT, GPTConfig

    per_token = GPT(GPTConfig.from_depth(2, sequence_len=32, vocab_size=256)).estimate_flops()
    budget = per_token * probe.total_batch_size * 3
    args = base + [f"--run-dir={run}", f"--target-flops={budget}", "--eval-every=3", "--eval-tokens=128", "--save-every=2"]
    assert base_train.main(args) == 0
    cfg = json.loads((run / "config.json").read_text())
    assert cfg["num_iterations"] == 3 and cfg["flops_per_token"] == per_token
    meta = json.loads(next((run / "checkpoints").glob("meta_000002*.json")).read_text())
    assert meta["loop_state"]["smooth_train_loss"] > 0 and meta["artifact_policy"] == "metrics_only"
    assert base_train.main(args + ["--resume-from-step=2"]) == 0
    rows = [json.loads(l) for l in open(run / "metrics_rank0.jsonl")]
    assert [r["step"] for r in rows if r["kind"] == "train"] == [1, 2, 3, 3]
    final = json.loads(next((run / "checkpoints").glob("meta_000003*.json")).read_text())
    assert final["val_bpb"] is not None and final["loop_state"]["min_val_bpb"] <= final["val_bpb"] + 1e-12


def test_research_policy_needs_pinned_inputs(tmp_path):
    with pytest.raises(SystemExit, match="research"):
        base_train.main(ARGS + [f"--run-dir={tmp_path}", "--artifact-policy=research"])
    with pytest.raises(SystemExit, match="needs --data-dir"):
        base_train.main(ARGS + [f"--run-dir={tmp_path}", f"--data-manifest={tmp_path / 'm.json'}"])


def test_fineweb_shards_with_a_verified_manifest(tmp_path):
    import numpy as np

    from archlab_b200.contracts import provenance as pv
    from archlab_b200.data.fineweb import write_fineweb_shard

    data = tmp_path / "data"
    data.mkdir()
    rng = np.random.default_rng(0)
    for name, n in (("fineweb_train_000001.bin", 700), ("fineweb_train_000002.bin", 500), ("fineweb_val_000000.bin", 400)):
        write_fineweb_shard(data / name, rng.integers(0, 256, n).astype(np.uint16))
    manifest = tmp_path / "manifest.json"
    pv.write_dataset_manifest(manifest, pv.create_dataset_manifest(data, dataset="toy-fineweb", revision="r0"))
    run = tmp_path / "run"
    args = ARGS + [f"--run-dir={run}", f"--data-dir={data}", f"--data-manifest={manifest}", "--data-verification=full",
                   "--eval-every=4", "--eval-tokens=128", "--no-final-checkpoint"]
    assert base_train.main(args) == 0
    cfg = json.loads((run / "config.json").read_text())
    assert cfg["data_identity"]["dataset"] == "toy-fineweb" and cfg["data_identity"]["mode"] == "full"
    rows = [json.loads(l) for l in open(run / "metrics_rank0.jsonl")]
    assert {r["data"] for r in rows if r["kind"] == "train"} == {"fineweb"} and sum(r["kind"] == "validation" for r in rows) == 2
    (data / "fineweb_val_000000.bin").write_bytes(b"tampered")
    with pytest.raises(pv.ProvenanceError):
        base_train.main(args)
