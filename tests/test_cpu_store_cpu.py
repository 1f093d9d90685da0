"""Host-resident tensor store over safetensors shards."""
import json

import pytest
import torch
from safetensors.torch import save_file

from archlab_b200.serve import cpu_store as cs


def _model(root):
    root.mkdir()
    g = torch.Generator().manual_seed(0)
    a = {"layers.0.ffn.experts.0.w": torch.randint(-128, 127, (6, 8), dtype=torch.int8, generator=g),
         "layers.0.ffn.experts.0.s": torch.rand(6, 1, generator=g).to(torch.float8_e4m3fn),
         "layers.0.attn.q": torch.randn(4, 4, generator=g).bfloat16(),
         "layers.0.ffn.experts.1.w": torch.randint(-128, 127, (6, 8), dtype=torch.int8, generator=g)}
    b = {"layers.1.ffn.experts.0.w": torch.randn(3, 5, generator=g).bfloat16(), "embed": torch.randn(10, 4, generator=g)}
    save_file(a, str(root / "a.safetensors"))
    save_file(b, str(root / "b.safetensors"))
    index = {"weight_map": {**{k: "a.safetensors" for k in a}, **{k: "b.safetensors" for k in b}}}
    (root / "model.safetensors.index.json").write_text(json.dumps(index))
    return {**a, **b}


def test_selected_tensors_are_resident_bit_for_bit(tmp_path):
    truth = _model(tmp_path / "m")
    events = []
    store = cs.ResidentTensorStore(tmp_path / "m", lambda n: ".ffn.experts." in n, threads=3, pinned=False, reserve_bytes=0, log=events.append)
    assert set(store.entries) == {n for n in truth if ".ffn.experts." in n} and "embed" not in store
    for name in store.entries:
        got, want = store.get(name), truth[name]
        assert got.dtype == want.dtype and got.shape == want.shape
        assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    assert store.report["tensors"] == 4 and store.report["shards"] == 2 and store.report["encoding_unchanged"]
    assert json.loads(events[0])["event"] == "host_store_ready"
    on_cpu = store.to_device(["layers.1.ffn.experts.0.w"], "cpu")
    assert torch.equal(on_cpu["layers.1.ffn.experts.0.w"], truth["layers.1.ffn.experts.0.w"])


def test_refusals(tmp_path):
    _model(tmp_path / "m")
    with pytest.raises(MemoryError, match="reserve"):
        cs.ResidentTensorStore(tmp_path / "m", lambda n: True, pinned=False, reserve_bytes=1 << 60)
    idx = tmp_path / "m" / "model.safetensors.index.json"
    doc = json.loads(idx.read_text())
    doc["weight_map"]["layers.0.attn.q"] = "../a.safetensors"
    idx.write_text(json.dumps(doc))
    with pytest.raises(ValueError, match="escapes"):
        cs.ResidentTensorStore(tmp_path / "m", lambda n: True, pinned=False, reserve_bytes=0)
    doc["weight_map"]["layers.0.attn.q"] = "a.safetensors"
    idx.write_text(json.dumps(doc))
    shard = tmp_path / "m" / "b.safetensors"
    shard.write_bytes(shard.read_bytes()[:-8])                       # truncated payload
    with pytest.raises(ValueError, match="exceeds its shard"):
        cs.ResidentTensorStore(tmp_path / "m", lambda n: True, pinned=False, reserve_bytes=0)
