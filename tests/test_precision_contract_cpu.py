"""Precision run contract, the FP4 geometry rules, and the block-scaled linear conversion with its BF16 exceptions."""
import pytest
import torch
import torch.nn as nn

from archlab_b200.ops import blockscaled as bs
from archlab_b200.train.precision_contract import check_fp4_geometry, precision_contract, resume_compatible


def test_contract_payloads():
    fp4 = precision_contract("fp4")
    assert fp4["stochastic_rounding"] and fp4["two_dimensional_quantization"] and fp4["dense_linear_alignment"] == 128
    assert fp4["moe_grouped_linear_max_experts"] == 64 and fp4["mtp_token_padding_multiple"] == 8
    assert "routing logits" in fp4["bf16_exceptions"]
    assert precision_contract("bf16")["mtp_token_padding_multiple"] == 1
    with pytest.raises(ValueError):
        precision_contract("int8")
    assert resume_compatible(precision_contract("bf16"), precision_contract("bf16")) == []
    assert "compute" in resume_compatible(precision_contract("bf16"), precision_contract("fp4"))


def test_fp4_geometry_rules():
    assert check_fp4_geometry(hidden_size=2048, intermediate_sizes=[512, 1408 + 128], num_experts=64, tokens_per_microbatch=8192, mtp_tokens=8) == []
    notes = check_fp4_geometry(hidden_size=1280, intermediate_sizes=[320], num_experts=128, tokens_per_microbatch=100, mtp_tokens=3)
    assert any(n.startswith("bf16:") and "320" in n for n in notes) and any("exceeds the cap" in n for n in notes)
    assert any("multiple of 64" in n for n in notes) and any("multiple of 8" in n for n in notes)


def test_conversion_reports_bf16_exceptions_and_runs_on_cpu():
    torch.manual_seed(0)
    m = nn.ModuleDict({"up": nn.Linear(128, 256, bias=False), "odd": nn.Linear(128, 192, bias=False), "router": nn.Linear(128, 128, bias=False),
                       "lm_head": nn.Linear(128, 512, bias=False), "biased": nn.Linear(128, 128)})
    rep = bs.convert_linears(m, "nvfp4")
    assert rep["converted"] == ["up"] and set(rep["bf16_exceptions"]) == {"odd", "router", "lm_head", "biased"}
    assert "not 128-aligned" in rep["bf16_exceptions"]["odd"]
    x = torch.randn(64, 128, requires_grad=True)
    y = m["up"](x)
    y.square().mean().backward()
    exact = x.detach() @ m["up"].weight.detach().t()
    assert (y.detach() - exact).norm() / exact.norm() < 0.2                 # the PyTorch statement of the FP4 products
    assert torch.isfinite(x.grad).all() and torch.isfinite(m["up"].weight.grad).all()
    gx = torch.autograd.grad((x @ m["up"].weight.t()).square().mean(), x)[0]
    assert (x.grad - gx).norm() / gx.norm() < 0.35
    bs.set_step(m, 7)
    assert m["up"].step == 7
    rep8 = bs.convert_linears(nn.ModuleDict({"a": nn.Linear(256, 128, bias=False)}), "fp8_block")
    assert rep8["converted"] == ["a"]
