"""Sealed window pilots: frozen selection, one label shift, exact masks, aligned empty batches."""
import json

import numpy as np
import pytest
import torch

from archlab_b200.data.sealed_windows import IGNORE, SealedWindows, seal_pilot


def corpus(root):
    root.mkdir()
    tokens = np.arange(1000, dtype=np.int32) % 97
    tokens.tofile(root / "part-00000.bin")
    (root / "DATA_READY.json").write_text(json.dumps({"parts": [{"file": "part-00000.bin", "tokens": 1000}]}))
    return root


WINDOWS = [{"part": "part-00000.bin", "start": 10, "length": 20, "assistant_label_spans": [[5, 9], [12, 20]], "targets": 12},
           {"part": "part-00000.bin", "start": 300, "length": 200, "assistant_label_spans": [[100, 200]], "targets": 100}]


def test_batches_carry_exact_masks_with_one_shift(tmp_path):
    src = corpus(tmp_path / "corpus")
    manifest = seal_pilot(tmp_path / "pilot", src, WINDOWS, split="train", context=256)
    assert manifest["supervised_tokens"] == 112
    data = SealedWindows(tmp_path / "pilot", expected_split="train", expected_budget=112, vocab_size=97)
    seen = 0
    for i in range(len(data)):
        x, y, n = data.batch(i)
        w = data.windows[i]
        assert x.shape == y.shape and x.shape[1] in (128, 256) and n == w["targets"]
        keep = y[0] != IGNORE
        source = torch.from_numpy((np.arange(1000) % 97)[w["start"]:w["start"] + w["length"] + 1].astype(np.int64))
        for lo, hi in w["assistant_label_spans"]:
            assert torch.equal(y[0, lo:hi], source[lo + 1:hi + 1])
        seen += n
    assert seen == 112
    x, y, n = data.batch(5)
    assert n == 0 and x.shape == (1, 128) and bool((y == IGNORE).all())
    assert data.batch(0, pad_to_full=True)[0].shape == (1, 256) and data.batch(9, pad_to_full=True)[0].shape == (1, 256)


def test_sealing_is_enforced(tmp_path):
    src = corpus(tmp_path / "corpus")
    seal_pilot(tmp_path / "pilot", src, WINDOWS, split="train", context=256)
    with pytest.raises(ValueError, match="wrong pilot format or split"):
        SealedWindows(tmp_path / "pilot", expected_split="heldout")
    with pytest.raises(ValueError, match="supervised-token budget"):
        SealedWindows(tmp_path / "pilot", expected_split="train", expected_budget=100)
    with pytest.raises(ValueError, match="invalid token window"):
        SealedWindows(tmp_path / "pilot", expected_split="train", vocab_size=50).batch(0)
    with pytest.raises(ValueError, match="spans do not add up"):
        seal_pilot(tmp_path / "bad", src, [{**WINDOWS[0], "targets": 11}], split="train", context=256)
    (src / "DATA_READY.json").write_text("{}")
    with pytest.raises(ValueError, match="source corpus changed"):
        SealedWindows(tmp_path / "pilot", expected_split="train")
    with (tmp_path / "pilot" / "windows.jsonl").open("a") as f:
        f.write("{}\n")
    with pytest.raises(ValueError, match="changed after sealing"):
        SealedWindows(tmp_path / "pilot", expected_split="train")
