"""Indexed-data trees: the files on disk must be exactly the declared parts."""
import json

import pytest

from archlab_b200.data.part_membership import data_prefixes, validated_data_prefixes


def tree(root, train=3, val=1):
    names = {"train_parts": [], "valid_parts": []}
    for split, key, n in (("train", "train_parts", train), ("val", "valid_parts", val)):
        (root / split).mkdir(parents=True)
        for i in range(n):
            for suffix in (".bin", ".idx", ".json"):
                (root / split / f"part-{i:05d}{suffix}").write_bytes(b"x")
            names[key].append(f"{split}/part-{i:05d}")
    (root / "DATA_READY.json").write_text(json.dumps(names))
    return names


def test_exact_membership(tmp_path):
    names = tree(tmp_path)
    train, val = validated_data_prefixes(tmp_path)
    assert [p.name for p in train] == ["part-00000", "part-00001", "part-00002"] and len(val) == 1
    names["valid_parts"] = [str((tmp_path / "val" / "part-00000").resolve())]              # absolute names are accepted too
    (tmp_path / "DATA_READY.json").write_text(json.dumps(names))
    assert validated_data_prefixes(tmp_path)[1] == val
    for suffix in (".bin", ".idx", ".json"):
        (tmp_path / "train" / f"part-00009{suffix}").write_bytes(b"x")
    with pytest.raises(RuntimeError, match="undeclared=.*part-00009"):
        validated_data_prefixes(tmp_path)
    (tmp_path / "train" / "part-00009.idx").write_bytes(b"")
    with pytest.raises(FileNotFoundError, match="missing or empty"):
        data_prefixes(tmp_path, "train")


def test_manifest_errors(tmp_path):
    names = tree(tmp_path)
    for edit, message in ((lambda n: n.update(train_parts=[]), "non-empty train_parts"), (lambda n: n.update(train_parts=n["train_parts"] + n["train_parts"][:1]), "duplicate"),
                          (lambda n: n.update(valid_parts=["val/part-00007"]), "missing=.*part-00007")):
        body = json.loads(json.dumps(names))
        edit(body)
        (tmp_path / "DATA_READY.json").write_text(json.dumps(body))
        with pytest.raises(RuntimeError, match=message):
            validated_data_prefixes(tmp_path)
    (tmp_path / "DATA_READY.json").write_text("[1]")
    with pytest.raises(RuntimeError, match="must hold an object"):
        validated_data_prefixes(tmp_path)
    (tmp_path / "DATA_READY.json").unlink()
    with pytest.raises(RuntimeError, match="invalid indexed-data manifest"):
        validated_data_prefixes(tmp_path)
