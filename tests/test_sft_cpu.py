import json

import pytest
import torch

from archlab_b200.ckpt.formats import state_sha256, verify_hf_export
from archlab_b200.data.tokenizer import BPETokenizer
from archlab_b200.models import limite as L
from archlab_b200.train import sft


def test_chat_rendering_masks_only_assistant_tokens_and_packing_never_splits():
    tok = BPETokenizer.train(["hello world how are you fine thanks"] * 4, 256 + 9 + 10)
    msgs = [{"role": "user", "content": "hello world"}, {"role": "assistant", "content": "fine thanks"}]
    ids, mask = sft.render_chat(tok, msgs)
    sp = tok.special
    a0, a1 = ids.index(sp["<|assistant_start|>"]), ids.index(sp["<|assistant_end|>"])
    assert sum(mask) == a1 - a0 and mask[a1] == 1 and mask[a0] == 0 and sum(mask[:a0]) == 0
    with pytest.raises(ValueError):
        sft.render_chat(tok, [{"role": "system", "content": "x"}])
    ex = [(list(range(1, 8)), [0, 0, 0, 1, 1, 1, 1]), (list(range(10, 16)), [0, 0, 1, 1, 1, 1]), (list(range(20, 24)), [0, 1, 1, 1])]
    x, y = sft.pack_examples(ex, 10)
    assert x.shape == (2, 10) and x[0, :6].tolist() == [1, 2, 3, 4, 5, 6] and x[1, :5].tolist() == [10, 11, 12, 13, 14]
    assert y[0, :6].tolist() == [-1, -1, 4, 5, 6, 7] and (y[0, 6:] == -1).all() and x[1, 5:8].tolist() == [20, 21, 22]


def test_sft_lowers_loss_and_export_carries_lineage(tmp_path):
    torch.manual_seed(0)
    cfg = L.LimiteConfig.tiny(vocab_size=64, num_hidden_layers=2)
    m = L.LimiteLM(cfg)
    m.init_weights(0.1)
    parent = state_sha256(m.state_dict())
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    x = torch.randint(0, 64, (4, 16))
    y = torch.roll(x, -1, 1)
    y[:, :8] = -1
    first = sft.sft_step(m, opt, x, y)
    for _ in range(30):
        last = sft.sft_step(m, opt, x, y)
    assert last["loss"] < first["loss"] - 0.5 and last["supervised_tokens"] == 32
    manifest = tmp_path / "manifest.json"
    manifest.write_text(json.dumps({"files": []}))
    sft.finalize_export(tmp_path / "export", m, {"arch_family": "limite", "hidden_size": 64}, stage="full_sft",
                        supervised_tokens=31 * 32, parent_state_sha256=parent, data_manifest=manifest)
    verify_hf_export(tmp_path / "export")
    lin = sft.read_lineage(tmp_path / "export")
    assert lin["parent_stage"] == "full_sft" and lin["parent_tokens"] == 992 and lin["parent_state_sha256"] == parent
    with pytest.raises(ValueError):
        sft.finalize_export(tmp_path / "e2", m, {}, stage="rl", supervised_tokens=1, parent_state_sha256=parent, data_manifest=manifest)
