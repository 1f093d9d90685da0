"""ZeroAdamW keeps fp32 main gradients for low-precision parameters: micro-batch accumulation is exact
in fp32 where a bf16 accumulator would round the small contributions away."""
import torch

from archlab_b200.optim.zero import ZeroAdamW


def test_bf16_parameters_accumulate_gradients_in_fp32():
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(8, 16).bfloat16())
    b = torch.nn.Parameter(torch.zeros(16).bfloat16())
    opt = ZeroAdamW([w, b], lr=1e-2, weight_decay=0.0)
    assert opt.main_grads and opt.flat_g.dtype == torch.float32 and w.grad is None
    before = w.detach().clone()
    # one large and many small contributions: bf16 accumulation would drop the small ones (2^-10 of the sum)
    x_big, x_small = torch.full((1, 8), 16.0).bfloat16(), torch.full((1, 8), 2.0 ** -6).bfloat16()
    expect = torch.zeros(8, 16)
    for x in [x_big] + [x_small] * 64:
        y = (x @ w + b).float().sum()
        y.backward()
        expect += x.float().t().expand(8, 16)
        assert w.grad is None                         # folded into the main gradient and dropped
    lo, hi = opt.range_of([w])
    main = opt.flat_g[lo:hi].view(8, 16)
    assert torch.equal(main, expect)
    bf16_sum = torch.zeros(8, 16).bfloat16()
    for x in [x_big] + [x_small] * 64:
        bf16_sum += x.t().expand(8, 16)
    assert not torch.equal(bf16_sum.float(), expect)  # the failure mode the fp32 buffer avoids
    opt.reduce_gradients()
    opt.step()
    assert not torch.equal(w.detach(), before) and float(opt.flat_g.abs().sum()) == 0.0


def test_fp32_parameters_keep_gradient_views():
    w = torch.nn.Parameter(torch.randn(4, 4))
    opt = ZeroAdamW([w], lr=1e-2)
    assert not opt.main_grads and w.grad.data_ptr() == opt.flat_g.data_ptr()
