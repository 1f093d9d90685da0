"""Adapter training on a frozen V4.1 backbone: input gradients only, and the numerics the frozen weights were released with.

``freeze_backbone(model)`` turns a ``V41LM`` into a fixed function of its inputs and of whatever trainable modules are
attached later (adapters, a new head):

* every ``QuantLinear`` keeps its parameter (checkpoint keys do not change) but computes through ``FrozenLinearFn``: the
  weight is block-rounded ONCE at installation, the forward is ``rounded(x) @ rounded(W)^T``, and the backward is the
  straight-through surrogate ``dX = dY @ rounded(W)`` -- the input activation is not saved, which is where the memory of a
  frozen backbone goes otherwise.  This is a training surrogate, not the derivative of rounding.
* every hyper-connection produces its coefficients through ``FrozenCoefficientsFn``: forward without a graph (optionally
  rounded to bf16 and carried as fp32, the precision of the released coefficient kernel), backward by re-running the
  PyTorch equations for d(mixes) only; scale and base are constants.
* routed and shared expert outputs are already summed in fp32 and rounded once by ``SparseMoE``; the installer checks
  that property on a probe instead of assuming it.

All base parameters end with ``requires_grad=False``; a second installation is refused; the returned receipt lists what
was changed.  (The reference installs the same three behaviours on an external implementation of the model:
src/archlab/automodel/deepseek_v41_autograd.py:21-57, deepseek_v41_official_hc.py:48-103, deepseek_v41_official_moe.py:1-10.)
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import quant
from .blocks import hc_split_sinkhorn
from .deepseek_v41 import HyperConnectionMix, QuantLinear, V41LM


class FrozenLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, rounded_weight, block):
        if rounded_weight.requires_grad:
            raise ValueError("the base weight must be frozen")
        ctx.save_for_backward(rounded_weight)                      # not x: the weight has no gradient to compute
        ctx.input_dtype = x.dtype
        xq = quant.rounded_activation(x.detach(), bits=8, block_size=block) if block and x.size(-1) % block == 0 else x.detach()
        return F.linear(xq, rounded_weight.to(x.dtype))

    @staticmethod
    def backward(ctx, dy):
        (w,) = ctx.saved_tensors
        return torch.matmul(dy.to(w.dtype), w).to(ctx.input_dtype), None, None


class FrozenCoefficientsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mixes, scale, base, streams, iterations, eps, carry_bf16):
        if scale.requires_grad or base.requires_grad:
            raise ValueError("hyper-connection scale and base must be frozen")
        ctx.save_for_backward(mixes, scale, base)
        ctx.geometry = (streams, iterations, eps)
        values = hc_split_sinkhorn(mixes, scale, base, streams, iterations, eps)
        if carry_bf16:
            values = tuple(v.bfloat16().float() for v in values)
        return values

    @staticmethod
    def backward(ctx, d_pre, d_post, d_comb):
        mixes, scale, base = ctx.saved_tensors
        with torch.enable_grad():
            x = mixes.detach().requires_grad_()
            (dx,) = torch.autograd.grad(hc_split_sinkhorn(x, scale, base, *ctx.geometry), x, (d_pre, d_post, d_comb))
        return dx, None, None, None, None, None, None


def _frozen_linear_forward(self, x):
    return FrozenLinearFn.apply(x, self._rounded_weight, self.block if self.fp8 else 0)


def _frozen_coefficients(self, streams):
    from .blocks import rms_norm

    flat = rms_norm(streams.flatten(-2).float(), eps=self.eps)
    mixes = F.linear(flat, self.proj.weight.float())
    scale, base = self.scale.detach().clone(), self.base.detach().clone()      # value copies: nothing aliases a sharded parameter
    if torch.is_grad_enabled() and mixes.requires_grad:
        return FrozenCoefficientsFn.apply(mixes, scale, base, self.n, self.iters, self.eps, self._carry_bf16)
    values = hc_split_sinkhorn(mixes, scale, base, self.n, self.iters, self.eps)
    return tuple(v.bfloat16().float() for v in values) if self._carry_bf16 else values


def _fp32_sum_probe(layer) -> bool:
    """True when routed and shared expert outputs are added in fp32 and rounded once: the layer's output must equal, bit
    for bit, the rounding of (fp32 routed subtotal + fp32 shared output) computed here from the layer's own parts."""
    from . import moe

    if getattr(layer, "shared", None) is None or not isinstance(layer, moe.SparseMoE):
        return True
    with torch.no_grad():
        x = torch.randn(8, layer.dim, device=layer.router.device, dtype=layer.router.dtype)
        w, idx, _ = moe.route(x, layer.router, layer.e_score_correction_bias, top_k=layer.top_k, score=layer.score, route_scale=layer.route_scale)
        tok = torch.arange(8, device=x.device).repeat_interleave(layer.top_k)
        routed = torch.zeros(8, layer.dim, dtype=torch.float32, device=x.device).index_add_(0, tok, layer.experts(x[tok], idx.flatten(), w.flatten()[:, None]).float())
        shared = layer.shared(x).float()
        if layer.shared_gate is not None:
            shared = shared * torch.sigmoid(layer.shared_gate(x).float())
        load = layer._cumulative_expert_load
        got = layer(x)
        layer._cumulative_expert_load = load                          # the probe must not count as routed traffic
    return bool(torch.equal(got, (routed + shared).to(x.dtype)))


def freeze_backbone(model: V41LM, *, carry_coefficients_bf16: bool = False) -> dict:
    if not isinstance(model, V41LM):
        raise TypeError("expected a V41LM")
    if getattr(model, "_frozen_backbone", False):
        raise ValueError("the backbone is already frozen")
    before = dict(model.named_parameters())
    linears, mixes = [], []
    for name, module in model.named_modules():
        if isinstance(module, QuantLinear):
            with torch.no_grad():
                w = module.weight
                if module.fp8 and w.shape[-1] % module.block == 0:
                    q, s = quant.fp8_weight_quantize_2d(w, module.block)
                    w = quant.fp8_weight_dequantize_2d(q, s, module.block).to(module.weight.dtype)
                module.register_buffer("_rounded_weight", w.detach().clone(), persistent=False)
            module.forward = _frozen_linear_forward.__get__(module)
            linears.append(name)
        elif isinstance(module, HyperConnectionMix):
            module._carry_bf16 = carry_coefficients_bf16
            module.coefficients = _frozen_coefficients.__get__(module)
            mixes.append(name)
    for p in model.parameters():
        p.requires_grad_(False)
    after = dict(model.named_parameters())
    if before.keys() != after.keys() or any(after[k] is not v for k, v in before.items()):
        raise RuntimeError("freezing changed a parameter or a checkpoint key")
    sums_ok = _fp32_sum_probe(model.layers[0].ffn)
    model._frozen_backbone = True
    return {"frozen_linears": linears, "frozen_hyper_connections": mixes, "coefficients_carried_as": "bf16-in-fp32" if carry_coefficients_bf16 else "fp32",
            "linear_backward": "dX = dY @ rounded(W); input not saved", "expert_sum": "fp32, rounded once" if sums_ok else "unverified",
            "parameters_preserved": True, "trainable_parameters": 0}


class FrozenHeadCrossEntropy(torch.autograd.Function):
    """Summed cross entropy through a FROZEN output head, chunk by chunk over tokens: the forward computes each chunk's
    logits, its loss and -- because the head has no gradient of its own -- the chunk's d(loss)/d(hidden) right away,
    then drops the logits.  Nothing vocabulary-sized survives the forward, and the backward is one multiplication by
    the incoming scalar.  Labels of -100 are ignored; a batch without any target still yields a zero gradient of the
    right shape, so every rank keeps taking part in the backward collectives
    (src/archlab/automodel/deepseek_v41_loss.py:1-40)."""

    @staticmethod
    def forward(ctx, hidden, labels, weight, chunk_tokens):
        if weight.requires_grad:
            raise ValueError("the output head must be frozen")
        flat, targets = hidden.reshape(-1, hidden.shape[-1]), labels.reshape(-1)
        grad = torch.zeros_like(flat)
        total = torch.zeros((), dtype=torch.float32, device=hidden.device)
        for start in range(0, flat.shape[0], chunk_tokens):
            y = targets[start:start + chunk_tokens]
            keep = y != -100
            if not bool(keep.any()):
                continue
            logits = F.linear(flat[start:start + chunk_tokens][keep], weight).float()
            logp = torch.log_softmax(logits, -1)
            total += -logp.gather(-1, y[keep, None]).sum()
            dlogits = logp.exp_()
            dlogits.scatter_add_(-1, y[keep, None], torch.full_like(dlogits[:, :1], -1.0))
            rows = torch.nonzero(keep, as_tuple=True)[0] + start
            grad[rows] = (dlogits.to(weight.dtype) @ weight).to(grad.dtype)
        ctx.save_for_backward(grad)
        ctx.shape = hidden.shape
        return total

    @staticmethod
    def backward(ctx, upstream):
        (grad,) = ctx.saved_tensors
        return (grad * upstream.to(grad.dtype)).view(ctx.shape), None, None, None
