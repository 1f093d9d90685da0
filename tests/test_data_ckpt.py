"""Data loaders and checkpoint bundle (CPU)."""
import json

import numpy as np
import pytest
import torch

from archlab_b200.ckpt import speedrun as ck
from archlab_b200.data.fineweb import FineWebBinaryLoader, inspect_fineweb_shard, write_fineweb_shard
from archlab_b200.data.synthetic import ZipfTokens
from archlab_b200.data.token_batches import BinaryTokenBatches, NativeTokenBatches, partition_prefixes


def test_fineweb_rank_slices_and_seek(tmp_path):
    rng = np.random.default_rng(0)
    for i, n in enumerate((5000, 7000), start=1):
        write_fineweb_shard(tmp_path / f"fineweb_train_{i:06d}.bin", rng.integers(0, 50000, n))
    assert inspect_fineweb_shard(tmp_path / "fineweb_train_000001.bin") == 5000
    loaders = [FineWebBinaryLoader(tmp_path, "train", 2, 64, rank=r, world_size=2, device="cpu") for r in range(2)]
    x0, y0 = next(loaders[0])
    x1, y1 = next(loaders[1])
    assert torch.equal(x0.flatten()[1:], y0.flatten()[:-1])
    assert y0.flatten()[-1] == x1.flatten()[0]          # contiguous global range, one-token overlap
    # exact resume: batch k from a fresh loader seeked to k equals the k-th batch of a streamed loader
    stream = FineWebBinaryLoader(tmp_path, "train", 2, 64, rank=1, world_size=2, device="cpu")
    batches = [next(stream)[0] for _ in range(60)]       # crosses a shard boundary
    for k in (0, 17, 38, 59):
        seek = FineWebBinaryLoader(tmp_path, "train", 2, 64, rank=1, world_size=2, device="cpu", start_batch_index=k)
        assert torch.equal(next(seek)[0], batches[k])
    bad = tmp_path / "fineweb_val_000000.bin"
    bad.write_bytes(b"\0" * 100)
    with pytest.raises(ValueError, match="header is shorter"):
        inspect_fineweb_shard(bad)
    # the cursor wraps around the epoch and a seek is closed-form (no shard in between is opened)
    table = stream.table
    assert table.batches == ((5000 - 1) // 256, (7000 - 1) // 256) and table.epoch_batches == 19 + 27
    wrapped = FineWebBinaryLoader(tmp_path, "train", 2, 64, rank=1, world_size=2, device="cpu", start_batch_index=46 + 17)
    assert torch.equal(next(wrapped)[0], batches[17]) and wrapped.state_dict()["batch_index"] == 64


def test_fineweb_inventory(tmp_path):
    from archlab_b200.data.fineweb import fixed_fineweb_validation_loader, inspect_fineweb_dataset

    rng = np.random.default_rng(2)
    for i in (1, 2, 3):
        write_fineweb_shard(tmp_path / f"fineweb_train_{i:06d}.bin", rng.integers(0, 50000, 1000 * i))
    write_fineweb_shard(tmp_path / "fineweb_val_000000.bin", rng.integers(0, 50000, 900))
    with pytest.raises(ValueError, match="complete inventory"):
        inspect_fineweb_dataset(tmp_path)
    rep = inspect_fineweb_dataset(tmp_path, expected_train_shards=3)
    assert rep["validated_train_tokens"] == 6000 and rep["complete_inventory"] and rep["validation_tokens"] == 900
    part = inspect_fineweb_dataset(tmp_path, required_train_tokens=2500)
    assert part["validated_train_shards"] == 2 and not part["complete_inventory"]
    with pytest.raises(ValueError, match="are required"):
        inspect_fineweb_dataset(tmp_path, required_train_tokens=7000)
    (tmp_path / "fineweb_train_000002.bin").unlink()
    with pytest.raises(ValueError, match="000002 is missing"):
        inspect_fineweb_dataset(tmp_path, required_train_tokens=2500)
    gen = fixed_fineweb_validation_loader(tmp_path, 2, 32, window_batches=3, device="cpu")
    first = [next(gen)[0] for _ in range(3)]
    again = [next(gen)[0] for _ in range(3)]
    assert all(torch.equal(a, b) for a, b in zip(first, again))


def test_token_batches_python_and_native_agree(tmp_path):
    rng = np.random.default_rng(1)
    prefixes = []
    for i in range(3):
        p = tmp_path / f"part{i}"
        rng.integers(0, 1000, 4000 + 100 * i).astype(np.int32).tofile(f"{p}.bin")
        prefixes.append(p)
    assert partition_prefixes(prefixes, 1, 2) == [prefixes[1]]
    with pytest.raises(ValueError, match="distinct"):
        partition_prefixes(prefixes, 0, 4)
    py = BinaryTokenBatches(prefixes, batch_size=4, sequence_len=128, start_batch=5, device="cpu")
    nat = NativeTokenBatches(prefixes, batch_size=4, sequence_len=128, start_batch=5, device="cpu")
    for _ in range(40):                                   # wraps every part cyclically
        a, b = next(py), next(nat)
        assert torch.equal(a["tokens"], b["tokens"]) and torch.equal(a["labels"], b["labels"])
        assert torch.equal(a["tokens"].flatten()[1:], a["labels"].flatten()[:-1])
    nat.close()
    rep = BinaryTokenBatches(prefixes, batch_size=2, sequence_len=64, start_batch=3, device="cpu",
                             repeat_window_batches=2)
    seq = [next(rep)["tokens"] for _ in range(6)]
    assert torch.equal(seq[0], seq[2]) and torch.equal(seq[1], seq[5]) and not torch.equal(seq[0], seq[1])


def test_zipf_tokens_are_deterministic_and_skewed():
    a = ZipfTokens(65536, 128, 8, seed=0, rank=0).block(3)
    b = ZipfTokens(65536, 128, 8, seed=0, rank=0).block(3)
    c = ZipfTokens(65536, 128, 8, seed=0, rank=1).block(3)
    assert torch.equal(a, b) and not torch.equal(a, c) and a.shape == (8, 129)
    assert (a < 100).float().mean() > 0.3 and int(a.max()) < 65536


def test_checkpoint_bundle_roundtrip_and_partial_rejection(tmp_path):
    from archlab_b200.models.nanochat import GPT, GPTConfig

    cfg = GPTConfig(sequence_len=32, vocab_size=128, n_layer=2, n_head=2, n_kv_head=2, n_embd=64)
    torch.manual_seed(0)
    m = GPT(cfg)
    m.init_weights()
    meta = {"step": 7, "model_config": {"sequence_len": 32, "vocab_size": 128, "n_layer": 2, "n_head": 2,
                                        "n_kv_head": 2, "n_embd": 64}}
    rng = ck.capture_rng_state()
    expected = torch.rand(3)
    for rank in range(2):
        ck.save_checkpoint(tmp_path, 7, m.state_dict(), {"rank": rank}, meta, rank=rank, rng_data=rng)
    rep = ck.verify_checkpoint_bundle(tmp_path, 7, world_size=2, require_rng=True)
    assert rep["optimizer_shards"] == 2 and len(rep["files"]) == 6
    assert ck.find_last_step(tmp_path) == 7
    ck.restore_rng_state(ck.load_rng_state(tmp_path, 7, "cpu", rank=1))
    assert torch.equal(torch.rand(3), expected)
    m2, meta2 = ck.build_model(tmp_path, 7, "cpu")
    for (k, a), (_, b) in zip(m.state_dict().items(), m2.state_dict().items()):
        assert torch.equal(a, b), k
    (tmp_path / "optim_000007_rank1.pt").unlink()
    with pytest.raises(RuntimeError, match="incomplete checkpoint"):
        ck.verify_checkpoint_bundle(tmp_path, 7, world_size=2)
    (tmp_path / "meta_000007.json").write_text(json.dumps({"step": 8}))
    with pytest.raises(RuntimeError, match="step mismatch"):
        ck.verify_checkpoint_bundle(tmp_path, 7, world_size=1)
