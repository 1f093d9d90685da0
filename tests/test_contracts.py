"""Contracts layer: recipes, layered specs, budgets, throughput protocol, failure taxonomy, launch
plans, experiment merge and science validators (all CPU)."""
import json

import pytest
import yaml

from archlab_b200.contracts import experiment as E
from archlab_b200.contracts import performance as P
from archlab_b200.contracts import research as R
from archlab_b200.contracts.launch import LaunchPlan
from archlab_b200.contracts.recipe import read_recipe, recipe_sha256, split_recipe_reference
from archlab_b200.contracts.spec import SpecError, load_experiment
from archlab_b200.contracts.substrate import atomic_write_json, classify_failure, sha256_file, transfer_plan


def test_recipe_catalog_requires_explicit_profile(tmp_path):
    cat = tmp_path / "c.yaml"
    cat.write_text(yaml.safe_dump({"profiles": {"a": {"x": 1}, "b": {"x": 2}}}))
    assert read_recipe(f"{cat}#b") == {"x": 2}
    with pytest.raises(ValueError, match="explicit #PROFILE"):
        read_recipe(cat)
    with pytest.raises(ValueError, match="unknown recipe profile"):
        read_recipe(f"{cat}#zzz")
    with pytest.raises(ValueError):
        split_recipe_reference("file.yaml#")
    assert recipe_sha256(f"{cat}#a") != recipe_sha256(f"{cat}#b")


def _spec(tmp_path, **extra):
    base = {"schema_version": 1, "name": "n", "backend": "speedrun", "variant": "baseline", "seed": 0}
    base.update(extra)
    p = tmp_path / "s.yaml"
    p.write_text(yaml.safe_dump(base))
    return p


def test_layered_spec_extends_and_cycles(tmp_path):
    (tmp_path / "defaults.yaml").write_text(yaml.safe_dump({"model": {"depth": 4, "width": 8}, "seed": 3}))
    child = _spec(tmp_path, extends=["defaults.yaml"], model={"depth": 20})
    spec = load_experiment(child)
    assert spec.model == {"depth": 20, "width": 8} and spec.seed == 0
    assert len(spec.source_files) == 2
    a, b = tmp_path / "a.yaml", tmp_path / "b.yaml"
    a.write_text(yaml.safe_dump({"extends": "b.yaml"}))
    b.write_text(yaml.safe_dump({"extends": "a.yaml"}))
    with pytest.raises(SpecError, match="cyclic"):
        load_experiment(a)


def test_spec_rejects_absolute_paths_and_partial_research_block(tmp_path):
    with pytest.raises(SpecError, match="portable"):
        load_experiment(_spec(tmp_path, paths={"data": "/abs/path"}))
    with pytest.raises(SpecError, match="both comparison and artifacts"):
        load_experiment(_spec(tmp_path, comparison={"regime": "controlled"}))
    ok = load_experiment(_spec(tmp_path, paths={"data": "env:DATA_ROOT"}, comparison={"regime": "scaling"},
                               artifacts={"mode": "research"}))
    assert ok.resolve_paths(environ={"DATA_ROOT": str(tmp_path)})["data"] == str(tmp_path.resolve())
    with pytest.raises(SpecError, match="not set"):
        ok.resolve_paths(environ={})


def test_budget_resolution_rules():
    r = R.resolve_training_budget("controlled", batch_tokens=1000, parameter_count=10, target_train_tokens=2999)
    assert r.steps == 2 and r.effective_training_tokens == 2000
    r = R.resolve_training_budget("scaling", batch_tokens=1000, parameter_count=100, tokens_per_parameter=26)
    assert r.steps == 3
    r = R.resolve_training_budget("fixed_compute", batch_tokens=10, parameter_count=5,
                                  algorithmic_flops_per_token=2.0, target_model_flops=99.0)
    assert r.steps == 4
    with pytest.raises(R.ContractError, match="do not mix"):
        R.resolve_training_budget("controlled", batch_tokens=10, parameter_count=5, target_train_tokens=100,
                                  tokens_per_parameter=2)
    with pytest.raises(R.ContractError, match="smaller than one"):
        R.resolve_training_budget("controlled", batch_tokens=10, parameter_count=5, target_train_tokens=9)
    with pytest.raises(R.ContractError, match="may not disable"):
        R.ArtifactPolicy.from_mapping({"mode": "research", "raw_metrics": False})
    with pytest.raises(R.ContractError, match="mismatch"):
        R.assert_paired_controls({"seed": 1}, {"seed": 2})


def test_throughput_protocol_and_contract(tmp_path):
    ts = [0.0] + [float(i) for i in range(1, 16)]
    ts[3] += 0.5
    s = P.summarize_step_timestamps(ts, tokens_per_step=100, protocol=P.ThroughputProtocol(warmup_steps=5))
    assert s["throughput_sample_intervals"] == 10 and s["median_step_seconds"] == 1.0
    assert s["steady_state_tokens_per_second"] == 100.0
    with pytest.raises(P.PerformanceError):
        P.summarize_step_timestamps([0, 1, 1], tokens_per_step=1)
    c = P.ThroughputContract(samples=5)
    base = P.throughput_receipt(c, [3.0, 3.1, 3.05, 3.0, 3.2])
    good = P.throughput_receipt(c, [3.1, 3.2, 3.1, 3.3, 3.1])
    bad = P.throughput_receipt(c, [4.0] * 5)
    assert P.check_throughput(c, good, base)["passed"]
    assert not P.check_throughput(c, bad, base)["passed"]
    other = P.throughput_receipt(P.ThroughputContract(samples=5, warmup=3), [3.0] * 5)
    with pytest.raises(P.PerformanceError, match="different contract"):
        P.check_throughput(c, other, base)


def test_failure_taxonomy_and_artifacts(tmp_path):
    assert classify_failure(FloatingPointError("Non-finite training loss")).category == "numerical"
    assert classify_failure(RuntimeError("CUDA out of memory")).category == "capacity"
    op = classify_failure(RuntimeError("NCCL watchdog timeout"))
    assert op.category == "operational" and op.retriable
    assert classify_failure(RuntimeError("device status word = 1")).category == "operational"
    assert classify_failure(ValueError("bad")).category == "contract"
    assert classify_failure(KeyError("x")).category == "unknown"
    target = tmp_path / "d" / "x.json"
    atomic_write_json(target, {"b": 1, "a": 2})
    assert json.loads(target.read_text()) == {"a": 2, "b": 1}
    assert not list(target.parent.glob(".*.tmp"))
    assert len(sha256_file(target)) == 64
    (tmp_path / "tree" / "sub").mkdir(parents=True)
    (tmp_path / "tree" / "sub" / "f.txt").write_text("x")
    dirs, files = transfer_plan(tmp_path / "tree", "/remote")
    assert str(dirs[0]) == "/remote" and files[0][1] == "/remote/sub/f.txt"


def test_launch_plan_shell_renders_env_tokens():
    plan = LaunchPlan("speedrun", ("torchrun", "--data", "env:DATA_ROOT", "a b"), env={"X": "1 2"})
    assert plan.shell() == "X='1 2' torchrun --data \"${DATA_ROOT}\" 'a b'"
    assert json.loads(plan.json())["backend"] == "speedrun"


def _recipe(tmp_path, **kw):
    body = {"name": "pilot", "parent_checkpoint": str(tmp_path / "ckpt"), "data_manifest": str(tmp_path / "m.json")}
    body.update(kw)
    p = tmp_path / "r.yaml"
    p.write_text(yaml.safe_dump(body))
    return p


def test_experiment_merge_overlays_overrides_and_settings(tmp_path):
    base = _recipe(tmp_path, settings={"actor_rollout_ref.rollout.n": 8})
    overlay = tmp_path / "o.yaml"
    overlay.write_text(yaml.safe_dump({"execution": "sync", "settings": {"data.train_batch_size": 4}}))
    e = E.read_experiment(base, ["native_context=131072", "settings.actor_rollout_ref.rollout.n=6",
                                 "throughput.samples=7"], overlays=[overlay])
    assert e.execution == "sync" and e.settings == {"actor_rollout_ref.rollout.n": 6, "data.train_batch_size": 4}
    assert e.throughput.samples == 7
    tree = E.compose_trainer(e)
    assert tree["actor_rollout_ref"]["rollout"]["n"] == 6 and tree["trainer"]["v1"]["trainer_mode"] == "sync"
    assert tree["trainer"]["experiment_name"] == "pilot"
    assert len(E.fingerprint(tree)) == 64
    with pytest.raises(ValueError, match="unknown configuration path"):
        E.compose_trainer(E.read_experiment(base, ["settings.actor_rollout_ref.rollout.nope=1"]))
    with pytest.raises(ValueError, match="key=value"):
        E.read_experiment(base, ["oops"])
    with pytest.raises(ValueError, match="missing mandatory"):
        p = tmp_path / "bad.yaml"
        p.write_text(yaml.safe_dump({"name": "x"}))
        E.read_experiment(p)


@pytest.mark.parametrize("override,message", [
    ("settings.algorithm.adv_estimator=gae", "requires GRPO"),
    ("settings.actor_rollout_ref.rollout.n=1", "multiple responses"),
    ("settings.algorithm.rollout_correction.rollout_is_threshold=3.0", "capped at 2"),
    ("settings.actor_rollout_ref.actor.use_kl_loss=true", "reference-policy KL"),
    ("settings.actor_rollout_ref.rollout.max_model_len=4096", "native context"),
    ("settings.data.truncation=left", "silently truncating"),
    ("settings.trainer.resume_mode=auto", "fresh RL must reset"),
    ("settings.actor_rollout_ref.actor.megatron.dtype=float16", "bfloat16"),
    ("settings.ray_kwargs.ray_init.runtime_env.env_vars.VERL_MFU_DEVICE_NAME=H100", "B200"),
])
def test_science_validators_fail_closed(tmp_path, override, message):
    base = _recipe(tmp_path)
    E.compose_trainer(E.read_experiment(base))          # the defaults are admissible
    with pytest.raises(ValueError, match=message):
        E.compose_trainer(E.read_experiment(base, [override]))


def test_experiment_cross_field_rules(tmp_path):
    with pytest.raises(ValueError, match="unknown model family"):
        E.read_experiment(_recipe(tmp_path, family="gpt9"))
    with pytest.raises(ValueError, match="primary execution engine"):
        E.read_experiment(_recipe(tmp_path, engine="dp"))
    with pytest.raises(ValueError, match="native control requires DP"):
        E.read_experiment(_recipe(tmp_path, family="qwen3_5", engine="dp"))
    with pytest.raises(ValueError, match="package SFT endpoint"):
        E.read_experiment(_recipe(tmp_path, intervention="replace_attention"))
    ok = E.read_experiment(_recipe(tmp_path, family="qwen3_5", engine="dp", attention="native", intervention="none",
                                   parent_stage="published_checkpoint", parent_tokens=None,
                                   publisher_manifest="m.json"))
    assert ok.family == "qwen3_5"
    with pytest.raises(ValueError, match="environment variable"):
        E.compose_trainer(E.read_experiment(_recipe(tmp_path, settings={"data.train_files": "${oc.env:NOPE_X}"})),
                          environ={})
    t = E.compose_trainer(E.read_experiment(_recipe(tmp_path, settings={"data.train_files": "${oc.env:D,/x}"})),
                          environ={})
    assert t["data"]["train_files"] == "/x"
