"""Block quantizers for the FP8 / NVFP4 training recipes (PyTorch statements; CPU oracles).

* ``fp8_block_quantize``: groups of ``block`` (128 or 32) along the last dim, scale = amax/448 with
  an optional exact power-of-two ceiling built from the exponent bits, e4m3 RNE cast
  (src/archlab/automodel/deepseek_v41_native_quantization.py:17-39).
* ``fp8_weight_quantize_2d``: 128 x 128 weight tiles, one scale per tile (V4.1-style training GEMM
  recipe: activations 1 x 128, weights 128 x 128).
* ``nvfp4_quantize``: e2m1 values in 16-element blocks with e4m3 block scales and one fp32
  per-tensor scale; round-to-nearest-even on the explicit codebook or stochastic rounding; optional
  random Hadamard transform (applied to both wgrad operands so it cancels in the product)
  (recipe in src/archlab/speedrun/precision.py:170-205; FP4 codebook / tie rule in
  src/archlab/architectures/deepseek_v41_torch.py:91-121).
* ``rounded_activation``: dequantised native-style activation rounding with a straight-through
  gradient.
* ``stochastic_bfloat16``: unbiased fp32 -> bf16 store (src/archlab/optimizers/sharded_adafactor.py:19-26).
"""
from __future__ import annotations

import math

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def pow2_ceil_scale(scales: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= each positive fp32 scale, from the exponent bits (no log2 rounding
    at exact exponent boundaries)."""
    bits = scales.contiguous().view(torch.int32)
    exponent = ((bits >> 23) & 255) + ((bits & ((1 << 23) - 1)) != 0)
    return (exponent << 23).view(torch.float32)


@torch.no_grad()
def fp8_block_quantize(x: torch.Tensor, block: int = 128, *, pow2: bool = True):
    """-> (e4m3 values with x's shape, fp32 scales [..., last/block])."""
    if block < 1 or x.ndim < 1 or x.shape[-1] % block:
        raise ValueError("FP8 activation width must divide its positive block size")
    g = x.float().unflatten(-1, (-1, block))
    s = g.abs().amax(-1).clamp_min(1e-4) * (1.0 / 448)
    if pow2:
        s = pow2_ceil_scale(s)
    q = (g / s.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.flatten(-2).contiguous(), s.contiguous()


def fp8_block_dequantize(q: torch.Tensor, s: torch.Tensor, block: int = 128) -> torch.Tensor:
    return (q.float().unflatten(-1, (-1, block)) * s.unsqueeze(-1)).flatten(-2)


@torch.no_grad()
def fp8_weight_quantize_2d(w: torch.Tensor, block: int = 128, *, pow2: bool = True):
    """[N, K] weight -> (e4m3 [N, K], fp32 scales [ceil(N/block), ceil(K/block)])."""
    N, K = w.shape
    pn, pk = (-N) % block, (-K) % block
    wp = torch.nn.functional.pad(w.float(), (0, pk, 0, pn))
    t = wp.view((N + pn) // block, block, (K + pk) // block, block)
    s = t.abs().amax(dim=(1, 3)).clamp_min(1e-4) * (1.0 / 448)
    if pow2:
        s = pow2_ceil_scale(s)
    q = (t / s[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(N + pn, K + pk)[:N, :K].contiguous(), s.contiguous()


def fp8_weight_dequantize_2d(q: torch.Tensor, s: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = q.shape
    full = s.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return q.float() * full


def _e2m1_round(z: torch.Tensor, *, stochastic: bool = False, generator=None) -> torch.Tensor:
    """Nearest (ties to even code) or stochastic rounding of |z| <= 6 onto the e2m1 grid."""
    book = torch.tensor(E2M1_VALUES, device=z.device, dtype=torch.float32)
    a = z.abs().clamp_max(6.0)
    if stochastic:
        hi_idx = torch.bucketize(a.contiguous(), book).clamp_max(7)          # first grid point >= a
        lo_idx = (hi_idx - 1).clamp_min(0)
        lo, hi = book[lo_idx], book[hi_idx]
        span = (hi - lo).clamp_min(1e-12)
        p_up = torch.where(hi > lo, (a - lo) / span, torch.zeros_like(a))
        u = torch.rand(a.shape, device=a.device, generator=generator)
        val = torch.where(u < p_up, hi, lo)
    else:
        bounds = torch.tensor(_E2M1_BOUNDS, device=z.device, dtype=torch.float32)
        codes = torch.bucketize(a.contiguous(), bounds)
        codes = codes + ((codes % 2 == 1) & (a == bounds[codes.clamp_max(6)])).long()
        val = book[codes]
    return torch.copysign(val, z)


def hadamard_matrix(n: int, device=None, dtype=torch.float32) -> torch.Tensor:
    if n & (n - 1):
        raise ValueError("Hadamard size must be a power of two")
    h = torch.ones(1, 1, device=device, dtype=dtype)
    while h.size(0) < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h / math.sqrt(n)


def random_hadamard_transform(x: torch.Tensor, sign: torch.Tensor, block: int = 16) -> torch.Tensor:
    """Blockwise x -> (x * sign) H over the last dim; orthogonal, so applying it to both operands of
    a contraction over that dim leaves the product unchanged while spreading outliers."""
    h = hadamard_matrix(block, x.device, torch.float32)
    g = (x.float() * sign.float()).unflatten(-1, (-1, block))
    return (g @ h).flatten(-2)


@torch.no_grad()
def nvfp4_quantize(x: torch.Tensor, block: int = 16, *, stochastic: bool = False, generator=None,
                   tensor_scale: torch.Tensor | None = None):
    """-> (dequantisable e2m1 values as fp32 on the grid, e4m3 block scales, fp32 tensor scale).

    ``x ~= values * block_scale.float() * tensor_scale``.  The tensor scale maps the global amax to
    the top of the representable range (6 * 448) so block scales use e4m3's range well."""
    if x.shape[-1] % block:
        raise ValueError("NVFP4 needs the last dimension to be a multiple of the block")
    xf = x.float()
    if tensor_scale is None:
        tensor_scale = (xf.abs().amax().clamp_min(1e-12) / (6.0 * 448.0)).reshape(())
    g = xf.unflatten(-1, (-1, block)) / tensor_scale
    bs = (g.abs().amax(-1, keepdim=True) / 6.0).clamp_min(2.0 ** -9).to(torch.float8_e4m3fn)
    z = (g / bs.float()).clamp(-6, 6)
    vals = _e2m1_round(z, stochastic=stochastic, generator=generator)
    return vals.flatten(-2), bs.squeeze(-1).contiguous(), tensor_scale


def nvfp4_dequantize(vals: torch.Tensor, block_scale: torch.Tensor, tensor_scale: torch.Tensor,
                     block: int = 16) -> torch.Tensor:
    return (vals.unflatten(-1, (-1, block)) * block_scale.float().unsqueeze(-1)).flatten(-2) * tensor_scale


class _IdentityGradient(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, rounded):
        return rounded

    @staticmethod
    def backward(ctx, g):
        return g, None


def rounded_activation(x: torch.Tensor, *, bits: int = 8, block_size: int = 32, e4m3_scale: bool = False,
                       straight_through: bool = True) -> torch.Tensor:
    if bits not in (4, 8) or block_size < 1 or x.shape[-1] % block_size:
        raise ValueError("unsupported activation quantization geometry")
    if bits == 8 and e4m3_scale:
        raise ValueError("native FP8 activations use power-of-two scales")
    with torch.no_grad():
        g = x.float().unflatten(-1, (-1, block_size))
        amax = g.abs().amax(-1, keepdim=True)
        if bits == 8:
            scale = pow2_ceil_scale(amax.clamp_min(1e-4) * (1.0 / 448))
            vals = (g / scale).clamp(-448, 448).to(torch.float8_e4m3fn).float()
        else:
            if e4m3_scale:
                scale = (amax.clamp_min(6 * 2 ** -9) / 6).to(torch.float8_e4m3fn).float()
            else:
                scale = pow2_ceil_scale(amax.clamp_min(6 * 2.0 ** -126) * (1.0 / 6))
            vals = _e2m1_round((g / scale).clamp(-6, 6))
        rounded = (vals * scale).flatten(-2).to(x.dtype)
    return _IdentityGradient.apply(x, rounded) if straight_through else rounded


def stochastic_bfloat16(value: torch.Tensor, *, generator=None) -> torch.Tensor:
    if value.dtype != torch.float32:
        raise TypeError("stochastic rounding takes FP32 values")
    noise = torch.randint(0, 65536, value.shape, dtype=torch.int32, device=value.device, generator=generator)
    bits = value.contiguous().view(torch.int32)
    return ((bits + noise) >> 16).to(torch.int16).view(torch.bfloat16)


def fp8_linear_reference(x: torch.Tensor, w: torch.Tensor, block: int = 128) -> torch.Tensor:
    """y = x W^T with 1 x block activation scales and block x block weight scales, fp32 accumulate:
    the numerical contract of the block-scaled FP8 training GEMM."""
    xq, xs = fp8_block_quantize(x, block)
    wq, ws = fp8_weight_quantize_2d(w, block)
    return fp8_block_dequantize(xq, xs, block) @ fp8_weight_dequantize_2d(wq, ws, block).t()
