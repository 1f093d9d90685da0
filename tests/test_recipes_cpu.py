"""Every shipped recipe loads through the loader of its schema."""
from pathlib import Path

import pytest

from archlab_b200.contracts import experiment as E
from archlab_b200.contracts.recipe import read_recipe
from archlab_b200.contracts.spec import load_experiment

ROOT = Path(__file__).resolve().parents[1] / "recipes"


@pytest.mark.parametrize("ref,backend", [("reference/speedrun.yaml#d20", "speedrun"), ("reference/speedrun.yaml#d20-simplicial", "speedrun"),
                                         ("reference/speedrun.yaml#d4-cpu", "speedrun"), ("reference/mesh.yaml#qwen35-4b-simplicial", "megatron"),
                                         ("reference/mesh.yaml#v41-moe-ep8", "megatron"), ("reference/mesh.yaml#qwen38-flash-next", "megatron")])
def test_layered_specs(ref, backend):
    s = load_experiment(ROOT / ref)
    assert s.backend == backend and s.parallelism["gpus_per_node"] >= 1 and s.training["sequence_length"] >= 256
    assert set(s.config["paths"]) == {"data_root", "run_dir"}


def test_inheritance_overrides_only_what_it_names():
    base, child = load_experiment(ROOT / "reference/speedrun.yaml#d20"), load_experiment(ROOT / "reference/speedrun.yaml#d20-simplicial")
    assert child.model["depth"] == base.model["depth"] == 20 and child.variant == "simplicial" and "simplicial_layers" in child.model


def test_rl_recipes_and_overlay(monkeypatch):
    monkeypatch.setenv("ARCHLAB_PARENT_CHECKPOINT", "/ckpt")
    monkeypatch.setenv("ARCHLAB_DATA_MANIFEST", "/m.json")
    e = E.read_experiment(ROOT / "rl/limite_code.yaml", [], overlays=[ROOT / "rl/limite_code_local.yaml"])
    assert e.execution == "colocate_async" and e.parent_checkpoint == "/ckpt"
    assert e.settings["data.train_batch_size"] == 8 and e.settings["actor_rollout_ref.rollout.n"] == 8
    assert E.read_experiment(ROOT / "rl/qwen35_code.yaml", []).engine == "dp"


def test_launch_catalog_and_study_contract():
    cat = read_recipe(f"{ROOT / 'qwen/launches.yaml'}#flash_next_quarter")
    assert cat["family"] == "flash-next" and cat["environment"]["NGA_FLASH_NEXT_MODEL_VARIANT"] == "quarter-depth48-no-mtp"
    with pytest.raises(ValueError):
        read_recipe(ROOT / "qwen/launches.yaml")
    assert read_recipe(ROOT / "deepseek_v41/scratch_w640_d20.yaml")["parallelism"]["expert"] == 8


@pytest.mark.parametrize("recipe,overlays", [("rl/limite_code.yaml", []), ("rl/limite_code.yaml", ["rl/limite_code_local.yaml"]),
                                             ("rl/qwen35_code.yaml", [])])
def test_rl_recipes_compose_and_pass_the_science_validators(monkeypatch, recipe, overlays):
    """The shipped RL recipes resolve against the packaged trainer tree: every settings path exists, the
    environment interpolations are filled in and the fail-closed pilot rules hold."""
    monkeypatch.setenv("ARCHLAB_PARENT_CHECKPOINT", "/ckpt/parent")
    monkeypatch.setenv("ARCHLAB_DATA_MANIFEST", "/data/manifest.json")
    exp = E.read_experiment(ROOT / recipe, overlays=[ROOT / o for o in overlays])
    assert exp.parent_checkpoint == "/ckpt/parent"
    tree = E.compose_trainer(exp)
    assert tree["trainer"]["experiment_name"] == exp.name
    assert tree["actor_rollout_ref"]["rollout"]["n"] == 8
    if overlays:
        assert tree["data"]["train_batch_size"] == 8 and tree["trainer"]["total_training_steps"] == 20
    # a broken rule is refused with its message
    exp.settings["actor_rollout_ref.rollout.n"] = 1
    with pytest.raises(ValueError):
        E.compose_trainer(exp)
