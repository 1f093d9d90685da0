"""SFT bootstrap contract: recipe, guarded settings, asset binding, immutable receipts."""
import json

import pytest
import torch
import yaml

from archlab_b200.ckpt.formats import export_hf
from archlab_b200.contracts.substrate import sha256_file
from archlab_b200.train import sft_bootstrap as sb


def world(tmp_path, *, conversion=True, rows=16):
    tok = tmp_path / "tok"
    tok.mkdir()
    (tok / "tokenizer.json").write_text(json.dumps({"model": {"vocab": {"a": 0}}}))
    (tok / "chat_template.jinja").write_text("{{ messages }}")
    config = {"vocab_size": 8, "eos_token_id": 7, "trainable_mode": "full", **({"conversion": {"short_window": 16}} if conversion else {})}
    export_hf(tmp_path / "parent", {"w": torch.ones(2, 2)}, config, tokenizer_dir=tok, lineage={"stage": "conversion"})
    data = tmp_path / "data"
    data.mkdir()
    (data / "train.jsonl").write_text("{}\n" * rows)
    (data / "validation.jsonl").write_text("{}\n")
    manifest = {"format": sb.DATA_FORMAT, "tokenization": {"loss_mask_alignment": "unshifted-target-token", "max_length": 4096, "generation_eos_token_id": 7,
                                                            "files": {n: sha256_file(tmp_path / "parent" / n) for n in ("tokenizer.json", "chat_template.jinja")}},
                "files": {"train": {"name": "train.jsonl", "sha256": sha256_file(data / "train.jsonl"), "rows": rows},
                          "validation": {"name": "validation.jsonl", "sha256": sha256_file(data / "validation.jsonl"), "rows": 1}}}
    (data / "manifest.json").write_text(json.dumps(manifest))
    recipe = {"name": "boot", "parent_checkpoint": str(tmp_path / "parent"), "data_manifest": str(data / "manifest.json"), "native_context": 8192,
              "settings": {"model.path": str(tmp_path / "parent"), "data.max_length": 4096, "data.train_files": [str(data / "train.jsonl")],
                           "data.val_files": [str(data / "validation.jsonl")]}}
    (tmp_path / "recipe.yaml").write_text(yaml.safe_dump(recipe))
    return tmp_path / "recipe.yaml"


def test_prepare_binds_parent_data_and_sources(tmp_path):
    recipe = world(tmp_path)
    (tmp_path / "pkg").mkdir()
    (tmp_path / "pkg" / "m.py").write_text("x = 1\n")
    receipt = sb.prepare(recipe, tmp_path / "out", package_root=tmp_path / "pkg")
    assert receipt["assets"]["variant"] == "simplicial" and receipt["settings"]["trainer"]["experiment_name"] == "boot"
    assert sb.prepare(recipe, tmp_path / "out", package_root=tmp_path / "pkg") == receipt                  # same receipt: accepted
    with pytest.raises(ValueError, match="already differs"):
        sb.prepare(recipe, tmp_path / "out", ["settings.data.train_batch_size=16"], package_root=tmp_path / "pkg")
    snapshot = json.loads((tmp_path / "out" / "source_snapshot.json").read_text())
    sb.verify_source(snapshot)
    (tmp_path / "pkg" / "m.py").write_text("x = 2\n")
    with pytest.raises(ValueError, match="changed after the freeze"):
        sb.verify_source(snapshot)


def test_settings_cannot_turn_the_experiment_into_something_else(tmp_path):
    recipe = world(tmp_path)
    for override, message in (("settings.engine.tensor_parallel=2", "data parallelism only"), ("settings.model.lora_rank=8", "full weights"),
                              ("settings.data.truncation=right", "un-truncated"), ("settings.data.train_batch_size=12", "whole number"),
                              ("settings.trainer.resume_mode=auto", "fresh experiment"), ("settings.data.max_length=9000", "native context"),
                              ("settings.model.path=/elsewhere", "explicit parent export"), ("objective=sequence_kd", "assistant-only"),
                              ("settings.optimizer.lr=1", "unknown settings section"), ("colour=red", "unknown bootstrap override")):
        with pytest.raises(ValueError, match=message):
            sb.compose_settings(sb.read_bootstrap(recipe, [override]))


def test_asset_mismatches_are_named(tmp_path):
    recipe = world(tmp_path)
    exp = sb.read_bootstrap(recipe)
    cfg = sb.compose_settings(exp)
    with pytest.raises(ValueError, match="conversion state differs"):
        sb.validate_assets(sb.read_bootstrap(recipe, ["variant=normal"]), cfg)
    with pytest.raises(ValueError, match="does not establish trained weights"):
        sb.validate_assets(sb.read_bootstrap(recipe, ["parent_stage=package_sft"]), cfg)
    data = tmp_path / "data"
    (data / "train.jsonl").write_text("{}\n" * 17)
    with pytest.raises(ValueError, match="data checksum mismatch: train"):
        sb.validate_assets(exp, cfg)
    (data / "train.jsonl").write_text("{}\n" * 16)
    manifest = json.loads((data / "manifest.json").read_text())
    manifest["tokenization"]["files"]["tokenizer.json"] = "0" * 64
    (data / "manifest.json").write_text(json.dumps(manifest))
    with pytest.raises(ValueError, match="tokenizer / template checksum differs"):
        sb.validate_assets(exp, cfg)
