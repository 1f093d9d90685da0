"""Model-only evaluation checkpoints: hard-linked payloads, filtered metadata, bitwise read-back, guarded retirement."""
import os

import pytest
import torch

from archlab_b200.ckpt.formats import save_megatron_dist
from archlab_b200.ckpt.model_only import export_model_only, is_model_key


def _save(root, iteration, seed=0):
    g = torch.Generator().manual_seed(seed + iteration)
    model = {"embedding.word_embeddings.weight": torch.randn(16, 8, generator=g), "decoder.layers.0.mlp.weight": torch.randn(8, 8, generator=g).bfloat16(),
             "output_layer.weight": torch.randn(16, 8, generator=g)}
    opt = {name: {"exp_avg": torch.zeros_like(t, dtype=torch.float32), "exp_avg_sq": torch.ones_like(t, dtype=torch.float32)} for name, t in model.items()}
    save_megatron_dist(root, iteration, model, opt, rng_state={"seed": 1})
    return model


def test_conversion_keeps_weight_bytes_and_drops_everything_else(tmp_path):
    import torch.distributed.checkpoint as dcp

    root = tmp_path / "run" / "checkpoints"
    model = _save(root, 10)
    _save(root, 20)
    receipt = export_model_only(root / "iter_0000010", tmp_path / "audit")
    stage = receipt["stage"]
    keys = list(dcp.FileSystemReader(stage).read_metadata().state_dict_metadata)
    assert sorted(keys) == sorted(model) and all(is_model_key(k) for k in keys)
    assert receipt["phase"] == "validated" and receipt["dropped_keys"] >= 7 and receipt["can_resume"] is False
    for row in receipt["files"]:
        assert os.stat(os.path.join(stage, row["file"])).st_ino == os.stat(root / "iter_0000010" / row["file"]).st_ino      # hard links
    got = {k: torch.empty_like(v) for k, v in model.items()}
    dcp.load(got, checkpoint_id=stage)
    assert all(torch.equal(got[k], model[k]) for k in model)
    assert export_model_only(root / "iter_0000010", tmp_path / "audit") == receipt                   # idempotent while validated
    done = export_model_only(root / "iter_0000010", tmp_path / "audit", retire=True)
    target = tmp_path / "run" / "eval-checkpoints" / "iter_0000010"
    assert done["phase"] == "complete" and not (root / "iter_0000010").exists() and (target / "EVAL_ONLY.json").exists()
    again = {k: torch.empty_like(v) for k, v in model.items()}
    dcp.load(again, checkpoint_id=str(target))
    assert all(torch.equal(again[k], model[k]) for k in model)                                       # links outlive the retired source


def test_refusals(tmp_path):
    root = tmp_path / "run" / "checkpoints"
    _save(root, 10)
    _save(root, 20)
    with pytest.raises(ValueError, match="latest checkpoint"):
        export_model_only(root / "iter_0000020", tmp_path / "audit")
    with pytest.raises(ValueError, match="protected"):
        export_model_only(root / "iter_0000010", tmp_path / "audit", protected_iterations=[10])
    (root / "notes").mkdir()
    with pytest.raises(ValueError, match="iteration checkpoint"):
        export_model_only(root / "notes", tmp_path / "audit")
    from archlab_b200.ckpt.formats import save_megatron_dist

    save_megatron_dist(root, 5, {"decoder.w": torch.ones(2)}, None)
    (root / "latest_checkpointed_iteration.txt").write_text("20")
    with pytest.raises(ValueError, match="no optimizer state"):
        export_model_only(root / "iter_0000005", tmp_path / "audit")
