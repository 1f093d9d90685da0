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


def test_pilot_selection_hits_the_budget_exactly_and_counts_every_target_once(tmp_path):
    from archlab_b200.data.sealed_windows import select_pilot_windows, shifted_window_spans

    assert shifted_window_spans([[3, 12]], 0, 8) == [[2, 8]] and shifted_window_spans([[3, 12]], 8, 8) == [[0, 3]]      # tokens 3..8 | 9..11
    assert shifted_window_spans([[3, 12]], 0, 8, limit=4) == [[2, 6]] and shifted_window_spans([[0, 2]], 0, 8) == [[0, 1]]   # token 0 has no predecessor
    with pytest.raises(ValueError, match="sorted"):
        shifted_window_spans([[5, 9], [2, 4]], 0, 8)
    src = corpus(tmp_path / "corpus")
    docs = [{"part": "part-00000.bin", "offset": 0, "tokens": 300, "assistant_token_spans": [[10, 40], [100, 290]]},
            {"part": "part-00000.bin", "offset": 300, "tokens": 200, "assistant_token_spans": [[50, 200]]},
            {"part": "part-00000.bin", "offset": 500, "tokens": 64, "assistant_token_spans": []}]
    windows, summary = select_pilot_windows(docs, target_tokens=333, context=128, seed=3)
    assert summary["supervised_tokens"] == 333 == sum(w["targets"] for w in windows) and summary["documents"] == 2
    seal_pilot(tmp_path / "pilot", src, windows, split="train", context=128)
    data = SealedWindows(tmp_path / "pilot", expected_split="train", expected_budget=333)
    assert sum(data.batch(i)[2] for i in range(len(data))) == 333
    all_windows, total = select_pilot_windows(docs, target_tokens=30 + 190 + 150, context=128)                           # every assistant token exactly once
    positions = sorted(w["start"] + lo + 1 + k for w in all_windows for lo, hi in w["assistant_label_spans"] for k in range(hi - lo))
    expected = sorted([p for a, b in [(10, 40), (100, 290)] for p in range(a, b)] + [300 + p for p in range(50, 200)])
    assert positions == expected and total["zero_target_windows_skipped"] <= 1       # the document without assistant text, if it came first
    with pytest.raises(ValueError, match="holds only"):
        select_pilot_windows(docs, target_tokens=10_000, context=128)
