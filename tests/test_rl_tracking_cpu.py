"""RL tracking: metric whitelist with ranges, exactly-once tailing of append-only ledgers."""
import json

import pytest

from archlab_b200.services import rl_tracking as rt
from archlab_b200.services.tracking import FileTrackingStore


def test_train_metrics_are_whitelisted_and_range_checked():
    row = {"update_step": 3, "reward_mean": 0.4, "reward_std": 0.1, "valid_answer_rate": 0.9, "skip_update": 0, "kl": 0.02, "policy_version": 3,
           "rollout_tokens": 5000, "rollout_seconds": 2.5, "secret_path": "/data/x", "nonflat_prompt_groups": 12}
    v = rt.train_values(row)
    assert v["rl/reward_mean"] == 0.4 and v["rl/kl"] == 0.02 and v["perf/rollout_tokens_per_second"] == 2000 and v["rl/policy_version"] == 3
    assert not any("secret" in k for k in v)
    assert "rl/kl" not in rt.train_values({**row, "reference_kl_available": False})
    for bad, message in (({"valid_answer_rate": 1.2}, r"\[0, 1\]"), ({"reward_std": -1}, "non-negative"), ({"nonflat_prompt_groups": 1.5}, "integer"),
                         ({"reward_mean": float("nan")}, "invalid scalar"), ({"update_skipped": 1, "skip_update": 0}, "conflicting aliases"),
                         ({"rollout_tokens": 10}, "positive rollout_seconds")):
        with pytest.raises(ValueError, match=message):
            rt.train_values(bad)
    with pytest.raises(ValueError, match="no recognised"):
        rt.train_values({"step": 1, "loss": 0.3})
    assert rt.evaluation_values({"pass_at_1": 0.25, "examples": 40})["eval/examples"] == 40
    with pytest.raises(ValueError, match="needs pass_at_1"):
        rt.evaluation_values({"examples": 40})
    with pytest.raises(ValueError, match="non-negative integer"):
        rt.update_step({"update_step": -1})


def test_profiles_publish_measured_scalars_only():
    profile = {"format": rt.PROFILE_FORMAT, "world_size": 8, "prompt_tokens": 512, "model_path": "/models/x",
               "batches": [{"batch_size_per_rank": 1, "generated_tokens_per_second": 900.0}, {"batch_size_per_rank": 4, "generated_tokens_per_second": 3100.0}]}
    v = rt.profile_values(profile)
    assert v["profile/batch_4/generated_tokens_per_second"] == 3100.0 and v["profile/world_size"] == 8 and not any("path" in k for k in v)
    with pytest.raises(ValueError, match="distinct"):
        rt.profile_values({**profile, "batches": profile["batches"] * 2})
    with pytest.raises(ValueError, match="unrecognised"):
        rt.profile_values({"format": "other"})


def test_ledgers_are_tailed_exactly_once(tmp_path):
    root = tmp_path / "run"
    root.mkdir()
    ledger = root / "metrics.jsonl"
    ledger.write_text(json.dumps({"update_step": 0, "reward_mean": 0.1, "time": 10}) + "\n" + json.dumps({"update_step": 1, "reward_mean": 0.2, "time": 11}) + "\n"
                      + '{"update_step": 2, "reward_m')                                              # a line still being written
    (root / "evaluation.jsonl").write_text(json.dumps({"step": 1, "pass_at_1": 0.5, "time": 12}) + "\n")
    (root / "rollout_profile.json").write_text(json.dumps({"format": rt.PROFILE_FORMAT, "world_size": 2}))
    store = FileTrackingStore(tmp_path / "store")
    sync = rt.RLMetricSync(store, tmp_path / "state.json")
    spec = {"source_id": "rl-run-1", "name": "grpo", "root": str(root), "tags": {"kind": "rl"}}
    first = sync.sync_run(spec)
    assert first["rows"] == {"train": 2, "evaluation": 1}
    points = [json.loads(l) for l in (tmp_path / "store" / first["run_id"] / "points.jsonl").read_text().splitlines()]
    assert ["rl/reward_mean", 0.2, 1, 11000] in points and ["eval/pass_at_1", 0.5, 1, 12000] in points and len(points) == 3
    assert json.loads((tmp_path / "store" / first["run_id"] / "meta.json").read_text())["params"]["profile/world_size"] == "2.0"
    with ledger.open("a") as f:
        f.write('ean": 0.3, "time": 13}\n')
    again = rt.RLMetricSync(store, tmp_path / "state.json").sync_run(spec)                               # a restarted sidecar resumes from its cursor
    assert again["rows"] == {"train": 1, "evaluation": 0} and again["run_id"] == first["run_id"]
    with ledger.open("a") as f:
        f.write(json.dumps({"update_step": 1, "reward_mean": 0.9}) + "\n")
    with pytest.raises(ValueError, match="went backwards"):
        sync.sync_run(spec)
    state = json.loads((tmp_path / "state.json").read_text())
    assert state["runs"]["rl-run-1"]["last_step"]["train"] == 2                                         # the refused line was not consumed
    ledger.write_text("")
    with pytest.raises(ValueError, match="append-only"):
        rt.RLMetricSync(store, tmp_path / "state.json").sync_run(spec)
