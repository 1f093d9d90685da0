"""Parquet shard stream: last shard is validation, ranks stride row groups, cursors resume exactly."""
import itertools

import pyarrow as pa
import pyarrow.parquet as pq
import pytest

from archlab_b200.data.parquet_shards import document_batches, list_shards, split_shards


def corpus(root, shards=3, groups=4, rows=2):
    root.mkdir()
    for s in range(shards):
        texts = [f"s{s}-g{g}-r{r}" for g in range(groups) for r in range(rows)]
        pq.write_table(pa.table({"text": texts}), root / f"shard_{s:05d}.parquet", row_group_size=rows)
    (root / "shard_00009.parquet.tmp").write_bytes(b"partial download")
    return root


def test_splits_and_rank_striding(tmp_path):
    root = corpus(tmp_path / "data")
    assert [p.name for p in list_shards(root)] == ["shard_00000.parquet", "shard_00001.parquet", "shard_00002.parquet"]
    assert [p.name for p in split_shards(root, "val")] == ["shard_00002.parquet"]
    seen = {r: [t for texts, _ in document_batches(root, "train", rank=r, world=2, epochs=1) for t in texts] for r in range(2)}
    assert not set(seen[0]) & set(seen[1]) and len(seen[0]) + len(seen[1]) == 2 * 4 * 2
    assert all(t.startswith(("s0", "s1")) for t in seen[0] + seen[1]) and seen[1][0] == "s0-g1-r0"
    val = [t for texts, _ in document_batches(root, "val", epochs=1) for t in texts]
    assert len(val) == 8 and all(t.startswith("s2") for t in val)
    with pytest.raises(ValueError):
        split_shards(root, "test")
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        list_shards(tmp_path / "empty")


def test_cursor_resumes_after_the_consumed_row_group_and_epochs_repeat(tmp_path):
    root = corpus(tmp_path / "data")
    full = list(itertools.islice(document_batches(root, "train", rank=1, world=2), 7))
    cursors = [c for _, c in full]
    assert cursors[:4] == [(0, 1, 1), (0, 3, 1), (1, 1, 1), (1, 3, 1)] and cursors[4] == (0, 1, 2)
    resumed = list(itertools.islice(document_batches(root, "train", rank=1, world=2, resume=cursors[2]), 4))
    assert [c for _, c in resumed] == cursors[3:7] and [t for t, _ in resumed] == [t for t, _ in full[3:7]]


def test_tokenizing_loader_resumes_exactly(tmp_path):
    import torch

    from archlab_b200.data.packing import tokenizing_loader

    root = corpus(tmp_path / "data", shards=3, groups=6, rows=3)

    class Tok:
        special = {"<|bos|>": 1}

        def encode(self, text):
            return [2 + (ord(c) % 23) for c in text]

    make = lambda **kw: tokenizing_loader(root, Tok(), 2, 8, buffer_size=6, **kw)
    run = make()
    history = [next(run) for _ in range(7)]
    assert all(bool((x[:, 0] == 1).all()) for x, _, _ in history) and history[4][2]["batch_index"] == 4
    assert history[-1][2]["shard"] >= history[0][2]["shard"] and history[0][2]["epoch"] == 1
    resumed = make(resume_state=history[4][2])
    x, y, state = next(resumed)
    assert torch.equal(x, history[4][0]) and torch.equal(y, history[4][1]) and state["batch_index"] == 4
    assert torch.equal(next(resumed)[0], history[5][0])
