"""Owner-aware loading of a released-name checkpoint: each rank fills exactly its experts; nothing is loaded best-effort."""
import json

import pytest
import torch

from archlab_b200.ckpt.ep_loading import expert_range, load_released_ep
from archlab_b200.ckpt.formats import export_v41_released


class Experts(torch.nn.Module):
    def __init__(self, n):
        super().__init__()
        self.gate_and_up_projs = torch.nn.Parameter(torch.zeros(n, 6, 8))
        self.down_projs = torch.nn.Parameter(torch.zeros(n, 4, 6))


class Tiny(torch.nn.Module):
    def __init__(self, n_experts):
        super().__init__()
        self.embed = torch.nn.Embedding(10, 6)
        self.layers = torch.nn.ModuleList()
        for _ in range(2):
            layer = torch.nn.Module()
            layer.ffn = torch.nn.Module()
            layer.ffn.experts = Experts(n_experts)
            layer.ffn.router = torch.nn.Linear(6, 4, bias=False)
            self.layers.append(layer)


def exported(tmp_path):
    torch.manual_seed(0)
    full = Tiny(4)
    for p in full.parameters():
        torch.nn.init.normal_(p)
    export_v41_released(tmp_path / "ckpt", list(full.state_dict().items()))
    return full, tmp_path / "ckpt"


def test_each_rank_loads_its_experts_and_all_replicated_tensors(tmp_path):
    full, ckpt = exported(tmp_path)
    assert list(expert_range(4, 1, 2)) == [2, 3]
    for rank in range(2):
        local = Tiny(2)
        report = load_released_ep(local, ckpt, ep_rank=rank, ep_size=2)
        assert report["counts"]["owned-expert-part"] == 2 * 2 * 3 and report["counts"]["remote-expert-part"] == 2 * 2 * 3
        for a, b in zip(local.layers, full.layers):
            assert torch.equal(a.ffn.experts.gate_and_up_projs, b.ffn.experts.gate_and_up_projs[2 * rank:2 * rank + 2])
            assert torch.equal(a.ffn.experts.down_projs, b.ffn.experts.down_projs[2 * rank:2 * rank + 2])
            assert torch.equal(a.ffn.router.weight, b.ffn.router.weight)
        assert torch.equal(local.embed.weight, full.embed.weight)
    whole = Tiny(4)
    load_released_ep(whole, ckpt, ep_rank=1, ep_size=2, local_experts=False)
    assert torch.equal(whole.layers[0].ffn.experts.down_projs[2:], full.layers[0].ffn.experts.down_projs[2:])
    assert float(whole.layers[0].ffn.experts.down_projs[:2].detach().abs().sum()) == 0


def test_strictness(tmp_path):
    full, ckpt = exported(tmp_path)
    index = json.loads((ckpt / "model.safetensors.index.json").read_text())
    with pytest.raises(ValueError, match="divisible"):
        load_released_ep(Tiny(2), ckpt, ep_rank=0, ep_size=3)
    with pytest.raises(ValueError, match="invalid checkpoint loading geometry"):
        load_released_ep(Tiny(2), ckpt, ep_rank=2, ep_size=2)
    with pytest.raises(FileNotFoundError):
        load_released_ep(Tiny(2), ckpt, ep_rank=0, ep_size=2, require_verified_copy=True)
    (ckpt / "VERIFIED_COPY.json").write_text(json.dumps({"source_index_sha256": "0" * 64}))
    with pytest.raises(ValueError, match="verified copy"):
        load_released_ep(Tiny(2), ckpt, ep_rank=0, ep_size=2, require_verified_copy=True)
    broken = {k: v for k, v in index["weight_map"].items() if not k.endswith("experts.1.w3.weight")}
    (ckpt / "model.safetensors.index.json").write_text(json.dumps({"weight_map": broken}))
    with pytest.raises(ValueError, match="owned expert parts are missing"):
        load_released_ep(Tiny(2), ckpt, ep_rank=0, ep_size=2)
    no_router = {k: v for k, v in index["weight_map"].items() if "router" not in k}
    (ckpt / "model.safetensors.index.json").write_text(json.dumps({"weight_map": no_router}))
    with pytest.raises(ValueError, match="missing model parameters"):
        load_released_ep(Tiny(2), ckpt, ep_rank=0, ep_size=2)
    escaped = dict(index["weight_map"])
    escaped[next(k for k in escaped if "router" in k)] = "../elsewhere.safetensors"
    (ckpt / "model.safetensors.index.json").write_text(json.dumps({"weight_map": escaped}))
    with pytest.raises(ValueError, match="direct children"):
        load_released_ep(Tiny(2), ckpt, ep_rank=0, ep_size=2)
