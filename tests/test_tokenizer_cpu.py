import pytest

from archlab_b200.data.tokenizer import BPETokenizer, core_metric


def test_train_round_trip_special_tokens_and_persistence(tmp_path):
    corpus = ["the quick brown fox jumps over the lazy dog " * 20, "hello world, hello there! 12345 ünïcödé \n\n tabs\tand spaces  "]
    tok = BPETokenizer.train(corpus, 256 + 9 + 40)
    assert tok.vocab_size == 305 and len(tok.merges) == 40
    for text in corpus + ["unseen words zebra 987", ""]:
        assert tok.decode(tok.encode(text)) == text
    assert len(tok.encode("the the the")) < len("the the the".encode())           # merges actually compress
    ids = tok.encode("<|user_start|>hi<|user_end|>", allow_special=True, prepend_bos=True)
    assert ids[0] == tok.special["<|bos|>"] and ids[1] == tok.special["<|user_start|>"] and ids[-1] == tok.special["<|user_end|>"]
    assert tok.special["<|user_start|>"] not in tok.encode("<|user_start|>")          # plain text unless allowed
    tb = tok.token_bytes()
    assert len(tb) == tok.vocab_size and tb[ord("a")] == 1 and tb[-1] == 0
    tok.save(tmp_path / "t.json")
    again = BPETokenizer.load(tmp_path / "t.json")
    assert again.sha256() == tok.sha256() and again.encode(corpus[1]) == tok.encode(corpus[1])
    assert BPETokenizer.train(corpus, 305).merges == tok.merges                       # deterministic
    (tmp_path / "bad.json").write_text((tmp_path / "t.json").read_text().replace('"merges": [[', '"merges": [[1, 2], ['))
    with pytest.raises(ValueError):
        BPETokenizer.load(tmp_path / "bad.json")


def test_core_metric():
    assert core_metric({"a": 0.5, "b": 0.25}, {"a": 0.5, "b": 0.25}) == 0.0
    assert core_metric({"a": 1.0, "b": 0.625}, {"a": 0.5, "b": 0.25}) == pytest.approx(0.75)
    with pytest.raises(ValueError):
        core_metric({"a": 1.0}, {"b": 0.5})
