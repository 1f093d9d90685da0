"""Publisher checkpoints are bound to a pinned manifest byte for byte."""
import json

import pytest

from archlab_b200.ckpt.publisher import REQUIRED_ASSETS, build_manifest, verify_publisher_checkpoint


def checkpoint(root):
    root.mkdir(parents=True)
    for name in REQUIRED_ASSETS - {"model.safetensors.index.json"}:
        (root / name).write_text(name)
    (root / "model-00001-of-00002.safetensors").write_bytes(b"a" * 32)
    (root / "model-00002-of-00002.safetensors").write_bytes(b"b" * 32)
    (root / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"w1": "model-00001-of-00002.safetensors", "w2": "model-00002-of-00002.safetensors"}}))
    return root


def test_a_pristine_copy_verifies_and_any_change_is_caught(tmp_path):
    root = checkpoint(tmp_path / "model")
    manifest = tmp_path / "pin.json"
    manifest.write_text(json.dumps(build_manifest(root, model_id="org/model", revision="a" * 40)))
    receipt = verify_publisher_checkpoint(root, manifest, model_id="org/model")
    assert receipt["shards"] == 2 and receipt["revision"] == "a" * 40 and len(receipt["files"]) == 8
    with pytest.raises(ValueError, match="pinned publisher manifest"):
        verify_publisher_checkpoint(root, manifest, model_id="org/other")
    (root / "tokenizer.json").write_text("tampered!!!!!")
    with pytest.raises(ValueError, match="bytes changed: tokenizer.json"):
        verify_publisher_checkpoint(root, manifest, model_id="org/model")
    (root / "tokenizer.json").write_text("tokenizer.json")
    (root / "EXPORT.json").write_text("{}")
    with pytest.raises(ValueError, match="experiment state"):
        verify_publisher_checkpoint(root, manifest, model_id="org/model")
    (root / "EXPORT.json").unlink()
    record = json.loads(manifest.read_text())
    short = dict(record, assets={k: v for k, v in record["assets"].items() if k != "model-00002-of-00002.safetensors"})
    manifest.write_text(json.dumps(short))
    with pytest.raises(ValueError, match="every weight shard"):
        verify_publisher_checkpoint(root, manifest, model_id="org/model")
    manifest.write_text(json.dumps(dict(record, publisher_revision="main")))
    with pytest.raises(ValueError, match="pinned publisher manifest"):
        verify_publisher_checkpoint(root, manifest, model_id="org/model")
    manifest.write_text(json.dumps(dict(record, assets={k: v for k, v in record["assets"].items() if k != "chat_template.jinja"})))
    with pytest.raises(ValueError, match="missing native"):
        verify_publisher_checkpoint(root, manifest, model_id="org/model")


def test_shared_weight_links_must_point_where_the_manifest_says(tmp_path):
    root = checkpoint(tmp_path / "model")
    store = tmp_path / "store"
    store.mkdir()
    shard = root / "model-00001-of-00002.safetensors"
    (store / "shard1").write_bytes(shard.read_bytes())
    shard.unlink()
    shard.symlink_to(store / "shard1")
    manifest = tmp_path / "pin.json"
    manifest.write_text(json.dumps(build_manifest(root, model_id="m", revision="b" * 40)))
    assert verify_publisher_checkpoint(root, manifest, model_id="m")["shards"] == 2
    (store / "other").write_bytes((store / "shard1").read_bytes())
    shard.unlink()
    shard.symlink_to(store / "other")                                     # same bytes, another target
    with pytest.raises(ValueError, match="symlink target changed"):
        verify_publisher_checkpoint(root, manifest, model_id="m")
