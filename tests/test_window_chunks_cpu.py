"""Document chunks: every target exactly once, no window across documents, receipts verified, exclusions honoured."""
import hashlib
import json

import numpy as np
import pytest

from archlab_b200.data.window_chunks import ChunkReader, document_windows, prepare_chunk


def encode_batch(texts):
    return [[10 + (ord(c) % 50) for c in t] for t in texts]


def test_windows_cover_each_target_once():
    assert list(document_windows(10, 4)) == [(0, 4), (4, 4), (8, 1)] and list(document_windows(5, 4)) == [(0, 4)]
    assert list(document_windows(2, 4)) == [(0, 1)] and list(document_windows(1, 4)) == []


def test_chunk_round_trip(tmp_path):
    texts = ["alpha beta gamma", "", "benchmark question", "x", "a much longer document than the window size allows in one piece"]
    exclude = frozenset({hashlib.sha256(b"benchmark question").hexdigest()})
    receipt = prepare_chunk(tmp_path, "train", 3, texts, encode_batch, sequence=8, exclude=exclude, source="part-3")
    assert receipt["documents"] == 3 and receipt["excluded_or_empty"] == 2 and receipt["targets"] == receipt["stored_tokens"] - receipt["documents"]
    assert prepare_chunk(tmp_path, "train", 3, ["changed"], encode_batch, sequence=8) == receipt          # finished chunks are not redone
    reader = ChunkReader(tmp_path / "chunks" / "train-000003")
    x, y = reader.batch(range(len(reader)))
    valid = y >= 0
    assert int(valid.sum()) == receipt["targets"] and x.shape == (receipt["windows"], 8)
    stream = np.fromfile(tmp_path / "chunks" / "train-000003" / "tokens.u32", dtype="<u4")
    targets = np.concatenate([row[m] for row, m in zip(y.numpy(), valid.numpy())])
    starts = np.flatnonzero(stream == 0)                                              # BOS marks document starts; BOS is never a target
    expected = np.delete(stream, starts)
    assert np.array_equal(targets, expected)
    for row_x, row_y, m in zip(x.numpy(), y.numpy(), valid.numpy()):
        assert 1 not in row_x[m].tolist()                                             # an EOD is never an input: no window crosses a document
    again = prepare_chunk(tmp_path / "other", "train", 3, texts, encode_batch, sequence=8, exclude=exclude, source="part-3")
    assert again["tokens_sha256"] == receipt["tokens_sha256"]                          # the shuffle depends on the chunk index only
    (tmp_path / "chunks" / "train-000003" / "tokens.u32").write_bytes(b"\0" * 8)
    with pytest.raises(ValueError, match="payload changed"):
        ChunkReader(tmp_path / "chunks" / "train-000003")
