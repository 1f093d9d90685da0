"""Launch recipes: allow-listed integer controls, family rules, environment overrides."""
import pytest
import yaml

from archlab_b200.contracts.launch_recipe import bindings, resolve_launch_recipe

BASE = {"NGA_EXPECTED_NODES": 2, "NGA_GPUS_PER_NODE": 8, "NGA_SEQUENCE_LENGTH": 8192, "NGA_MICRO_BATCH_SIZE": 1, "NGA_GLOBAL_BATCH_SIZE": 256,
        "NGA_TARGET_TRAIN_TOKENS": 10_000_000_000, "NGA_CHECKPOINT_INTERVAL_TOKENS": 500_000_000, "NGA_PROBE_STEPS": 4}


def write(tmp_path, family="flash-next", **env):
    values = {**BASE, **({"NGA_FLASH_NEXT_MODEL_VARIANT": "1b-depth48-no-mtp", "NGA_PROBE_SAVE_INTERVAL": 2} if family == "flash-next" else
                         {"NGA_MODEL_SCALE": "quarter", "NGA_RUNTIME_PREFLIGHT": 1, "NGA_PREFLIGHT_STEPS": 3}), **env}
    path = tmp_path / f"{family}.yaml"
    path.write_text(yaml.safe_dump({"schema_version": 1, "family": family, "environment": {k: v for k, v in values.items() if v is not None}}))
    return path


def test_resolution_and_overrides(tmp_path):
    path = write(tmp_path)
    out = resolve_launch_recipe(path, {"NGA_GLOBAL_BATCH_SIZE": "0512", "UNRELATED": "x", "NGA_FLASH_NEXT_MODEL_VARIANT": "1b-depth48-no-mtp"})
    assert out["NGA_GLOBAL_BATCH_SIZE"] == "512" and out["NGA_EXPECTED_NODES"] == "2" and out["NGA_LAUNCH_FAMILY"] == "flash-next"
    assert len(out["NGA_LAUNCH_RECIPE_SHA256"]) == 64 and "UNRELATED" not in out
    lines = bindings(out).splitlines()
    assert lines == sorted(lines) and "NGA_GLOBAL_BATCH_SIZE=512" in lines
    dense = resolve_launch_recipe(write(tmp_path, "dense-27b"), {})
    assert dense["NGA_MODEL_SCALE"] == "quarter" and dense["NGA_RUNTIME_PREFLIGHT"] == "1"


def test_refusals(tmp_path):
    cases = [({"NGA_FLASH_NEXT_MODEL_VARIANT": "tiny"}, {}, "explicitly select a supported model"), ({"NGA_MODEL_SCALE": "full"}, {}, "mixes unrelated"),
             ({}, {"NGA_FLASH_NEXT_MODEL_VARIANT": "full"}, "conflicts with the recipe"), ({}, {"NGA_SEQUENCE_LENGTH": "8k"}, "unsigned decimal"),
             ({}, {"NGA_SEQUENCE_LENGTH": str(2 ** 63)}, "64-bit"), ({"NGA_MICRO_BATCH_SIZE": 0}, {}, "positive topology"),
             ({"NGA_PROBE_SAVE_INTERVAL": None}, {}, "every pre-flight / probe control"), ({"PATH": "/bin"}, {}, "unsupported environment keys")]
    for env, environment, message in cases:
        with pytest.raises(ValueError, match=message):
            resolve_launch_recipe(write(tmp_path, **env), environment)
    with pytest.raises(ValueError, match="positive number of steps"):
        resolve_launch_recipe(write(tmp_path, "dense-27b", NGA_PREFLIGHT_STEPS=0), {})
    with pytest.raises(ValueError, match="0 or 1"):
        resolve_launch_recipe(write(tmp_path, "dense-27b", NGA_RUNTIME_PREFLIGHT=2), {})
    bad = tmp_path / "bad.yaml"
    bad.write_text(yaml.safe_dump({"schema_version": 1, "family": "flash-next", "environment": {}, "extra": 1}))
    with pytest.raises(ValueError, match="exactly schema_version"):
        resolve_launch_recipe(bad, {})


def test_every_profile_of_the_shipped_launch_catalog_resolves():
    from pathlib import Path

    catalog = Path(__file__).resolve().parents[1] / "recipes" / "qwen" / "launches.yaml"
    profiles = yaml.safe_load(catalog.read_text())["profiles"]
    assert profiles
    for name in profiles:
        out = resolve_launch_recipe(f"{catalog}#{name}", {})
        assert out["NGA_LAUNCH_FAMILY"] in ("dense-27b", "flash-next") and int(out["NGA_EXPECTED_NODES"]) >= 1
    one, other = list(profiles)[0], list(profiles)[-1]
    assert resolve_launch_recipe(f"{catalog}#{one}", {})["NGA_LAUNCH_RECIPE_SHA256"] != resolve_launch_recipe(f"{catalog}#{other}", {})["NGA_LAUNCH_RECIPE_SHA256"]
