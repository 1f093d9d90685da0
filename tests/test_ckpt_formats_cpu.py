"""Checkpoint / export layouts: Megatron torch + torch_dist, HF safetensors, V4.1 sharded + released names, receipts."""
import json

import pytest
import torch

from archlab_b200.ckpt import formats as F


def _state():
    g = torch.Generator().manual_seed(0)
    return {"embedding.word_embeddings.weight": torch.randn(32, 8, generator=g),
            "decoder.layers.0.mlp.weight": torch.randn(8, 8, generator=g).bfloat16(),
            "decoder.final_norm.weight": torch.ones(8)}


def test_megatron_torch_layout(tmp_path):
    st = _state()
    F.save_megatron_torch(tmp_path, 12, st, {"step": 12}, rng_state={"seed": 0})
    assert (tmp_path / "latest_checkpointed_iteration.txt").read_text() == "12"
    assert (tmp_path / "iter_0000012" / "mp_rank_00" / "model_optim_rng.pt").is_file()
    assert F.validate_megatron_torch(tmp_path) == {"format": "torch", "iteration": 12, "shards": 1}
    F.save_megatron_torch(tmp_path, 13, st, None)
    with pytest.raises(ValueError):
        F.validate_megatron_torch(tmp_path)
    assert F.validate_megatron_torch(tmp_path, require_optimizer=False)["iteration"] == 13


def test_megatron_dist_layout_roundtrip(tmp_path):
    st = _state()
    opt = {n: {"exp_avg": torch.zeros_like(t, dtype=torch.float32), "exp_avg_sq": torch.ones_like(t, dtype=torch.float32)}
           for n, t in st.items()}
    d = F.save_megatron_dist(tmp_path, 7, st, opt, rng_state=torch.arange(4, dtype=torch.uint8))
    assert (d / ".metadata").is_file() and (d / "common.pt").is_file() and list(d.glob("*.distcp"))
    info = F.validate_megatron_dist(tmp_path)
    assert info["format"] == "torch_dist" and info["iteration"] == 7
    template = {k: torch.zeros_like(v) for k, v in st.items()}
    F.load_megatron_dist(tmp_path, template)
    for k in st:
        assert torch.equal(template[k], st[k])
    F.save_megatron_dist(tmp_path / "noopt", 1, st)
    with pytest.raises(ValueError):
        F.validate_megatron_dist(tmp_path / "noopt")


def test_hf_export_receipt_and_tamper(tmp_path):
    st = _state()
    r = F.export_hf(tmp_path, st, {"architectures": ["ArchlabForCausalLM"], "hidden_size": 8}, extra_files={"tokenizer.json": b"{}"},
                    lineage={"parent": "x"})
    assert r["format"] == "archlab-hf-v1" and set(r["files"]) == {"config.json", "model.safetensors", "tokenizer.json"}
    assert F.verify_hf_export(tmp_path)["state_sha256"] == F.state_sha256(st)
    (tmp_path / "config.json").write_text("{}")
    with pytest.raises(ValueError):
        F.verify_hf_export(tmp_path)


def test_v41_sharded_inventory_and_reconstruction(tmp_path):
    g = torch.Generator().manual_seed(1)
    state = {"embed_tokens.weight": torch.randn(37, 4, generator=g).bfloat16(),
             "layers.0.ffn.experts.gate_and_up_projs": torch.randn(8, 4, 6, generator=g),
             "layers.0.ffn.experts.down_projs": torch.randn(8, 3, 4, generator=g),
             "norm.weight": torch.ones(4)}
    F.write_v41_sharded(tmp_path, state, cursor={"step": 5, "tokens": 100}, replicated={"norm.weight"}, chunk_elements=7)
    inv = F.V41CheckpointInventory(tmp_path)
    rep = inv.report()
    assert rep["layouts"] == {"row16": 1, "expert_ep8_fsdp2": 2, "replicated": 1} and rep["tensor_count"] == 4
    for name, t in state.items():
        assert torch.equal(inv.read_tensor(name), t), name
    with pytest.raises(ValueError):
        inv.read_tensor("embed_tokens.weight", max_bytes=8)
    man = tmp_path / "rank-03" / "MANIFEST.json"
    data = json.loads(man.read_text())
    data["cursor"] = {"step": 6, "tokens": 100}
    man.write_text(json.dumps(data))
    with pytest.raises(ValueError):
        F.V41CheckpointInventory(tmp_path)
    assert F.shard_extent(37, 16, 0) == (0, 3) and F.shard_extent(37, 16, 12) == (36, 1)
    assert F.shard_extent(37, 16, 15) == (37, 0)


def test_v41_shard_extents_of_axes_the_piece_count_does_not_divide(tmp_path):
    """Ceil-width pieces with a short or empty tail, which is the placement a reference-written
    checkpoint has (src/archlab/serving/v41_checkpoint_inventory.py:20-23)."""
    assert [F.shard_extent(10, 4, i) for i in range(4)] == [(0, 3), (3, 3), (6, 3), (9, 1)]
    assert [F.shard_extent(3, 2, i) for i in range(2)] == [(0, 2), (2, 1)]
    assert [F.shard_extent(5, 4, i) for i in range(4)] == [(0, 2), (2, 2), (4, 1), (5, 0)]
    g = torch.Generator().manual_seed(3)
    state = {"embed_tokens.weight": torch.randn(10, 4, generator=g),
             "layers.0.ffn.experts.gate_and_up_projs": torch.randn(3, 5, 6, generator=g),
             "layers.0.ffn.experts.down_projs": torch.randn(3, 3, 5, generator=g)}
    F.write_v41_sharded(tmp_path, state, cursor={"step": 1, "tokens": 8}, world_size=4, ep_size=2,
                        expert_fsdp_size=2, engram_owners=4, chunk_elements=5)
    inv = F.V41CheckpointInventory(tmp_path)
    rows = [e["shape"][0] for e in inv.entries["embed_tokens.weight"]]
    assert rows == [3, 3, 3, 1]
    experts = [e["shape"][:2] for e in inv.entries["layers.0.ffn.experts.gate_and_up_projs"]]
    assert experts == [[2, 3], [1, 3], [2, 2], [1, 2]]      # rank = ep index + 2 * fsdp index
    for name, t in state.items():
        assert torch.equal(inv.read_tensor(name), t), name


def test_v41_released_name_export(tmp_path):
    from safetensors.torch import load_file

    E, C, I = 2, 4, 3
    tensors = [("embed_tokens.weight", torch.randn(10, C)), ("layers.0.ffn.experts.gate_and_up_projs", torch.randn(E, C, 2 * I)),
               ("layers.0.ffn.experts.down_projs", torch.randn(E, I, C)), ("layers.0.ffn.e_score_correction_bias", torch.zeros(E)),
               ("layers.0.engram.table", torch.randn(10, 2))]
    done = F.export_v41_released(tmp_path, tensors, engram_row_block=4)
    idx = json.loads((tmp_path / "model.safetensors.index.json").read_text())["weight_map"]
    assert done["tensors"] == len(idx) == 1 + 2 * E + E + 1 + 3
    assert "embed.weight" in idx and "layers.0.ffn.gate.bias" in idx and "layers.0.engram.table.rows.8" in idx
    w1 = load_file(str(tmp_path / idx["layers.0.ffn.experts.1.w1.weight"]))["layers.0.ffn.experts.1.w1.weight"]
    torch.testing.assert_close(w1, tensors[1][1][1, :, :I].t())
    w2 = load_file(str(tmp_path / idx["layers.0.ffn.experts.0.w2.weight"]))["layers.0.ffn.experts.0.w2.weight"]
    assert w2.shape == (C, I)
    assert len((tmp_path / "export-manifest.jsonl").read_text().splitlines()) == done["tensors"]


def test_run_receipts(tmp_path):
    r = F.RunReceipts(tmp_path / "a", {"name": "x"})
    r.log({"step": 1, "loss": 2.0})
    assert (tmp_path / "a" / "RUNNING.json").is_file()
    r.finish({"loss": 1.0})
    assert (tmp_path / "a" / "COMPLETE.json").is_file() and not (tmp_path / "a" / "RUNNING.json").exists()
    with pytest.raises(FileExistsError):
        F.RunReceipts(tmp_path / "a", {})
    f = F.RunReceipts(tmp_path / "b", {})
    f.finish(error=RuntimeError("CUDA out of memory"))
    failed = json.loads((tmp_path / "b" / "FAILED.json").read_text())
    assert "out of memory" in failed["error"] and failed["classification"]


def test_export_carries_the_tokenizer_and_checks_its_identity(tmp_path):
    import json

    import pytest
    import torch

    from archlab_b200.ckpt import formats

    tok = tmp_path / "tok"
    tok.mkdir()
    (tok / "tokenizer.json").write_text(json.dumps({"model": {"vocab": {"a": 0, "b": 1}}, "added_tokens": [{"id": 5, "content": "<eod>"}]}))
    (tok / "tokenizer_config.json").write_text("{}")
    (tok / "unrelated.bin").write_bytes(b"x")
    identity = formats.tokenizer_identity(tok)
    assert formats.tokenizer_vocab_size(tok) == 6
    state = {"w": torch.ones(2, 2)}
    receipt = formats.export_hf(tmp_path / "out", state, {"vocab_size": 8}, tokenizer_dir=tok, tokenizer_identity_sha256=identity)
    assert receipt["tokenizer_identity_sha256"] == identity
    assert {"tokenizer.json", "tokenizer_config.json"} <= set(receipt["files"]) and "unrelated.bin" not in receipt["files"]
    assert formats.tokenizer_identity(tmp_path / "out") == identity           # the export is self-contained
    formats.verify_hf_export(tmp_path / "out")
    with pytest.raises(ValueError, match="not the tokenizer"):
        formats.export_hf(tmp_path / "o2", state, {"vocab_size": 8}, tokenizer_dir=tok, tokenizer_identity_sha256="0" * 64)
    with pytest.raises(ValueError, match="embedding only"):
        formats.export_hf(tmp_path / "o3", state, {"vocab_size": 4}, tokenizer_dir=tok)
    (tok / "tokenizer.json").unlink()
    with pytest.raises(ValueError, match="needs tokenizer.json"):
        formats.export_hf(tmp_path / "o4", state, {"vocab_size": 8}, tokenizer_dir=tok)


def test_export_copy_is_verified_and_marked_last(tmp_path):
    import json

    import pytest
    import torch

    from archlab_b200.ckpt import formats

    tok = tmp_path / "tok"
    tok.mkdir()
    (tok / "tokenizer.json").write_text(json.dumps({"model": {"vocab": {"a": 0}}}))
    formats.export_hf(tmp_path / "export", {"w": torch.ones(2, 2)}, {"vocab_size": 4}, tokenizer_dir=tok)
    body = formats.copy_export(tmp_path / "export", tmp_path / "bulk" / "export")
    names = {f["path"] for f in body["files"]}
    assert {"config.json", "tokenizer.json", "model.safetensors", "EXPORT.json"} <= names
    assert json.loads((tmp_path / "bulk" / "export" / formats.COPY_MARKER).read_text()) == body
    formats.verify_hf_export(tmp_path / "bulk" / "export")
    (tmp_path / "export" / "config.json").write_text("{}")                          # a later change of the source is not picked up:
    assert formats.copy_export(tmp_path / "export", tmp_path / "bulk" / "export") == body      # the marked copy is final
    (tmp_path / "bulk" / "export" / formats.COPY_MARKER).unlink()                  # an unmarked destination is copied again
    again = formats.copy_export(tmp_path / "export", tmp_path / "bulk" / "export")
    assert (tmp_path / "bulk" / "export" / "config.json").read_text() == "{}" and again != body
    (tmp_path / "partial").mkdir()
    (tmp_path / "partial" / "config.json").write_text("{}")
    with pytest.raises(RuntimeError, match="source export is incomplete"):
        formats.copy_export(tmp_path / "partial", tmp_path / "bulk" / "partial")
