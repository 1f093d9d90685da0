"""Document windows: verified corpora, group-separated splits, windows inside documents, reproducible streams."""
import json

import numpy as np
import pytest

from archlab_b200.data.document_windows import MixtureWindows, Source, heldout_group, write_corpus

TOK = {"tokenizer.json": "a" * 64}


def corpus(path, n_docs=60, base=0, seed=0):
    rng = np.random.default_rng(seed)
    docs = [np.full(int(rng.integers(4, 40)), base + i, dtype=np.int32) for i in range(n_docs)]      # every token names its document
    return write_corpus(path, docs, [f"task-{i // 3}" for i in range(n_docs)], TOK), docs


def test_windows_stay_inside_documents_and_splits_follow_groups(tmp_path):
    m1, docs = corpus(tmp_path / "a")
    m2, _ = corpus(tmp_path / "b", base=1000, seed=1)
    data = MixtureWindows([Source(str(m1), 3.0), Source(str(m2), 1.0)], 8, tokenizer_files=TOK, vocab_size=2000, heldout_fraction=0.3)
    r = data.receipts[0]
    assert r["train_documents"] + r["heldout_documents"] + r["short_documents"] == 60 and r["short_documents"] == sum(len(d) < 8 for d in docs)
    rng = np.random.default_rng(0)
    train, held = data.sample(rng, 400), data.sample(rng, 200, heldout=True)
    assert train.shape == (400, 8) and bool((train == train[:, :1]).all()) and bool((held == held[:, :1]).all())
    train_docs, held_docs = set(train[:, 0].tolist()), set(held[:, 0].tolist())
    assert not train_docs & held_docs
    group = lambda d: f"task-{(d % 1000) // 3}"
    assert all(not heldout_group(group(d), 42, 0.3) for d in train_docs) and all(heldout_group(group(d), 42, 0.3) for d in held_docs)
    share = float((train[:, 0] < 1000).float().mean())
    assert 0.65 < share < 0.85                                                   # mixture weights 3 : 1
    a, b = data.rank_batch(7, 5, 1, 4), data.rank_batch(7, 5, 1, 4)
    assert bool((a == b).all()) and not bool((a == data.rank_batch(7, 5, 2, 4)).all())


def test_corpora_are_verified_before_use(tmp_path):
    m, _ = corpus(tmp_path / "a")
    kw = dict(tokenizer_files=TOK, vocab_size=100)
    with pytest.raises(ValueError, match="tokenizer identity"):
        MixtureWindows([Source(str(m))], 8, tokenizer_files={"tokenizer.json": "b" * 64}, vocab_size=100)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        MixtureWindows([Source(str(m))], 8, tokenizer_files=TOK, vocab_size=10)
    with pytest.raises(ValueError, match="both the train and the held-out"):
        MixtureWindows([Source(str(m))], 39, **kw)
    with pytest.raises(ValueError, match="positive finite weight"):
        Source(str(m), 0.0)
    body = json.loads(m.read_text())
    (tmp_path / "a" / "groups.json").write_text(json.dumps(["x"] * 60))
    with pytest.raises(ValueError, match="checksum differs"):
        MixtureWindows([Source(str(m))], 8, **kw)
    body["format"] = "tokens-only"
    m.write_text(json.dumps(body))
    with pytest.raises(ValueError, match="unsupported corpus format"):
        MixtureWindows([Source(str(m))], 8, **kw)
    with pytest.raises(ValueError, match="one group per"):
        write_corpus(tmp_path / "c", [np.arange(3)], [], TOK)
