"""Linear layers routed through the GEMM entry point: forward and both gradients against ``F.linear``."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from archlab_b200.ops.native_linear import NativeLinear, convert_linears, native_linear


def test_forward_and_gradients_match_f_linear():
    torch.manual_seed(0)
    x = torch.randn(3, 5, 16, requires_grad=True)
    w = torch.randn(24, 16, requires_grad=True)
    dy = torch.randn(3, 5, 24)
    native_linear(x, w).backward(dy)
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    F.linear(x, w).backward(dy)
    torch.testing.assert_close(native_linear(x, w), F.linear(x, w), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(gx, x.grad, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(gw, w.grad, atol=1e-5, rtol=1e-5)


def test_convert_keeps_parameters_and_skips_ineligible_layers():
    m = nn.Sequential(nn.Linear(128, 256, bias=False), nn.ReLU(), nn.Linear(256, 130, bias=False), nn.Linear(130, 8, bias=True))
    before = [p for p in m.parameters()]
    names = convert_linears(m)
    assert names == ["0"] and isinstance(m[0], NativeLinear) and type(m[2]) is nn.Linear
    assert all(a is b for a, b in zip(before, m.parameters()))
    x = torch.randn(4, 128)
    ref = nn.Sequential(nn.Linear(128, 256, bias=False), nn.ReLU(), nn.Linear(256, 130, bias=False), nn.Linear(130, 8, bias=True))
    ref.load_state_dict(m.state_dict())
    torch.testing.assert_close(m(x), ref(x), atol=1e-5, rtol=1e-5)


def test_trainer_flag_converts_the_factory_model(tmp_path, monkeypatch):
    from archlab_b200.train import mesh_train

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    base = ["--model=factory:nanochat", "--n-layer=2", "--model-set=n_embd=128", "--model-set=n_head=2", "--model-set=n_kv_head=2",
            "--model-set=vocab_size=512", "--seq-len=32", "--global-batch=2", "--micro-batch=2", "--steps=3"]
    plain = mesh_train.train(mesh_train.parse_args(base + [f"--run-dir={tmp_path / 'a'}"]))
    native = mesh_train.train(mesh_train.parse_args(base + ["--native-linears", f"--run-dir={tmp_path / 'b'}"]))
    assert all(abs(a - b) < 1e-4 for a, b in zip(plain, native)), (plain, native)
