"""Every trainable model family answers the same protocol."""
import pytest
import torch

from archlab_b200.models.protocol import check_protocol


def build(name):
    torch.manual_seed(0)
    if name == "v41":
        from archlab_b200.models.deepseek_v41 import V41Config, V41LM
        m = V41LM(V41Config.tiny())
    elif name == "qwen38":
        from archlab_b200.models.qwen38 import Qwen38Config, Qwen38LM
        m = Qwen38LM(Qwen38Config.for_scale("tiny"))
    elif name == "limite":
        from archlab_b200.models.limite import LimiteConfig, LimiteLM
        m = LimiteLM(LimiteConfig.tiny())
    elif name == "nanochat":
        from archlab_b200.models.nanochat import GPT, GPTConfig
        m = GPT(GPTConfig(sequence_len=32, vocab_size=64, n_layer=2, n_head=2, n_kv_head=2, n_embd=32))
    elif name == "sota":
        from archlab_b200.models.sota import SotaConfig, SotaLM
        m = SotaLM(SotaConfig())
    else:
        from archlab_b200.models.frontier import FrontierConfig, FrontierLM
        m = FrontierLM(FrontierConfig())
    m.init_weights()
    return m


@pytest.mark.parametrize("name", ["v41", "qwen38", "limite", "nanochat", "sota", "frontier"])
def test_protocol(name):
    m = build(name)
    report = check_protocol(m)
    assert report["parameters"] > 0 and report["flops_per_token"] > 6 * 0.2 * report["parameters"]
    assert m.get_architecture_state()["step"] == 3


def test_sparse_models_execute_fewer_flops_and_report_router_state():
    m = build("v41")
    ids = torch.randint(0, 256, (2, 16))
    m(ids, ids)
    assert m.estimate_executed_flops() < m.estimate_flops()
    state = m.get_architecture_state()
    assert state["expert_load"]["layers"] == 2 and 0 < state["expert_load"]["max_share"] <= 1
    metrics = m.consume_training_metrics()
    assert "cross entropy" in metrics and "router aux loss" in metrics and m.consume_training_metrics().get("cross entropy") is None
    contract = m.optimizer_contract()
    assert any(".experts." in n for n in contract["muon"]) and any("embed" in n for n in contract["adamw"])
