"""FP8 linear arithmetic (quantise, scaled products, gradients) on the CPU path, and module conversion."""
import torch

from archlab_b200.ops import fp8


def test_quantisation_round_trip_and_linear_gradients():
    torch.manual_seed(0)
    x = torch.randn(64, 48)
    q, inv = fp8.quantize_tensorwise(x)
    assert q.dtype == torch.float8_e4m3fn and (q.float() * inv - x).abs().max() < 0.07 * x.abs().max()
    lin, ref = fp8.Float8Linear(48, 32, bias=False), torch.nn.Linear(48, 32, bias=False)
    ref.weight.data.copy_(lin.weight.data)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya, yb = lin(xa), ref(xb)
    g = torch.randn_like(ya)
    ya.backward(g)
    yb.backward(g)
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    assert rel(ya, yb) < 0.06 and rel(xa.grad, xb.grad) < 0.12 and rel(lin.weight.grad, ref.weight.grad) < 0.12


def test_convert_linears_keeps_head_and_small_layers():
    m = torch.nn.ModuleDict({"a": torch.nn.Linear(256, 256, bias=False), "lm_head": torch.nn.Linear(256, 512, bias=False),
                             "small": torch.nn.Linear(16, 16, bias=False), "b": torch.nn.Sequential(torch.nn.Linear(256, 128, bias=False))})
    w = m["a"].weight
    assert fp8.convert_linears(m) == 2
    assert isinstance(m["a"], fp8.Float8Linear) and m["a"].weight is w and type(m["lm_head"]) is torch.nn.Linear
    assert type(m["small"]) is torch.nn.Linear and isinstance(m["b"][0], fp8.Float8Linear)
