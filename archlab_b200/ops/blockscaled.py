"""Block-scaled FP8 / NVFP4 operands and GEMMs on the tcgen05 ``block_scale`` path.

A ``ScaledOperand`` is a quantised matrix in the layout the tensor core consumes: data bytes row-major along
K plus scale factors in 512-byte chunks (``csrc/gemm_bs.h``).  Two formats:

``fp8``   e4m3 / e5m2 with one power-of-two (ue8m0) scale per 32 elements.  ``block=128`` gives the
          DeepSeek-V4.1 activation rule (1 x 128), ``block=-128`` its weight rule (128 x 128 blocks)
          (src/archlab/architectures/deepseek_v41_torch.py:91-121,
          src/archlab/automodel/deepseek_v41_native_quantization.py:17-39); both are this format with the
          scale repeated over the sub-blocks.
``nvfp4`` e2m1 pairs with one e4m3 scale per 16 elements and an fp32 tensor scale, optional 16 x 16 weight blocks,
          random Hadamard transform and stochastic rounding: the controls of the reference's NVFP4 recipe
          (src/archlab/speedrun/precision.py:170-205: RHT on, stochastic rounding on, 2-D weight quantisation).

Every function has a PyTorch statement of the same arithmetic (``decode``, ``reference_gemm``) that the GPU tests
compare against and that runs when no GPU is present.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import native

_vp, _i, _ll, _f, _u = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_uint
native.register_signature("nga_sf_bytes", [_i, _ll, _ll], _ll)
native.register_signature("nga_quant_mxfp8", [_vp, _vp, _vp, _ll, _ll, _ll, _ll, _i, _i, _vp])
native.register_signature("nga_quant_nvfp4", [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _i, _u, _u, _vp])
native.register_signature("nga_gemm_mxfp8", [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _i, _i, _i, _i,
                                             _f, _f, _vp, _vp])
native.register_signature("nga_gemm_nvfp4", [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _i, _i,
                                             _f, _f, _vp, _vp, _vp, _vp])
native.register_signature("nga_gemm_grouped_bs", [_i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _f, _vp, _vp,
                                                  _vp, _vp])

E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
NVFP4_RANGE = 448.0 * 6.0


@dataclass
class ScaledOperand:
    kind: str                     # "fp8" | "nvfp4"
    data: torch.Tensor            # uint8 [rows, K] (fp8) or [rows, K // 2] (fp4, element 2i in the low nibble)
    sf: torch.Tensor              # uint8, chunked scale factors
    rows: int
    K: int
    e5m2: bool = False
    amax: torch.Tensor | None = None     # nvfp4: fp32 scalar tensor, absolute maximum of the source tensor

    @property
    def chunk_span(self) -> int:
        return 128 if self.kind == "fp8" else 64

    @property
    def chunks_k(self) -> int:
        kblock = 128 if self.kind == "fp8" else 256
        return -(-self.K // kblock) * (kblock // self.chunk_span)


def sf_bytes(kind: str, rows: int, K: int) -> int:
    span, kblock = (128, 128) if kind == "fp8" else (64, 256)
    return -(-rows // 128) * (-(-K // kblock) * (kblock // span)) * 512


def sf_index(rows: int, n_sf: int, chunks_k: int, device=None) -> torch.Tensor:
    """Byte offset of scale (r, j) in the chunked array, as an int64 tensor [rows, n_sf]."""
    r = torch.arange(rows, device=device).view(-1, 1)
    j = torch.arange(n_sf, device=device).view(1, -1)
    rr = r % 128
    return ((r // 128) * chunks_k + j // 4) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + j % 4


def _pow2_scale_exponent(amax: torch.Tensor, fmax: float) -> torch.Tensor:
    """Smallest integer e with max(amax, 1e-4) / 2^e <= fmax, clamped to ue8m0's range; the floor is the one of the
    DeepSeek-V4.1 quantiser (src/archlab/automodel/deepseek_v41_native_quantization.py:31)."""
    safe = amax.float().clamp_min(1e-4).double()
    e = torch.ceil(torch.log2(safe / fmax))
    e = torch.where(torch.ldexp(torch.full_like(safe, fmax), e.int()) < safe, e + 1, e)
    e = torch.where(torch.ldexp(torch.full_like(safe, fmax), e.int() - 1) >= safe, e - 1, e)
    return e.clamp(-127, 127).to(torch.int32)


# ------------------------------------------------------------------------------------------------
# PyTorch statements (reference / CPU path)
# ------------------------------------------------------------------------------------------------
def quantize_fp8_reference(x: torch.Tensor, block: int = 32, e5m2: bool = False) -> ScaledOperand:
    rows, K = x.shape
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    fmax = torch.finfo(dt).max
    Kp = -(-K // 128) * 128
    xf = torch.zeros(rows, Kp, dtype=torch.float32, device=x.device)
    xf[:, :K] = x.float()
    if block == -128:
        Rp = -(-rows // 128) * 128
        pad = torch.zeros(Rp, Kp, dtype=torch.float32, device=x.device)
        pad[:rows] = xf
        amax = pad.view(Rp // 128, 128, Kp // 128, 128).abs().amax(dim=(1, 3))
        e = _pow2_scale_exponent(amax, fmax)                                    # [Rp/128, Kp/128]
        e_rows = e.repeat_interleave(128, 0)[:rows].repeat_interleave(4, 1)     # [rows, Kp/32]
    else:
        amax = xf.view(rows, Kp // abs(block), abs(block)).abs().amax(-1)
        e = _pow2_scale_exponent(amax, fmax)
        e_rows = e.repeat_interleave(abs(block) // 32, 1)
    inv = torch.ldexp(torch.ones_like(xf), -e_rows.repeat_interleave(32, 1))
    q = (xf * inv).clamp(-fmax, fmax).to(dt)[:, :K].contiguous()
    n_sf = Kp // 32
    sf = torch.zeros(sf_bytes("fp8", rows, K), dtype=torch.uint8, device=x.device)
    sf[sf_index(rows, n_sf, n_sf // 4, x.device).view(-1)] = (e_rows + 127).to(torch.uint8).view(-1)
    return ScaledOperand("fp8", q.view(torch.uint8), sf, rows, K, e5m2)


def _e2m1_encode(a: torch.Tensor, u: torch.Tensor | None) -> torch.Tensor:
    """|a| (already scaled) -> 3-bit code on the e2m1 grid; nearest-even, or stochastic with uniforms ``u``."""
    grid = torch.tensor(E2M1_GRID, device=a.device)
    a = a.clamp(max=6.0)
    lo = (a.unsqueeze(-1) >= grid[1:]).sum(-1)
    top = lo == 7
    lo_c = lo.clamp(max=6)
    frac = (a - grid[lo_c]) / (grid[lo_c + 1] - grid[lo_c])
    if u is not None:
        up = u < frac
    else:
        up = (frac > 0.5) | ((frac == 0.5) & (lo_c % 2 == 1))
    return torch.where(top, lo, lo_c + up.long())


def hadamard16(seed: int, device=None) -> torch.Tensor:
    """The sign-randomised 16 x 16 Hadamard matrix the quantiser applies to every 16-block (row vector times M)."""
    h = torch.ones(1, 1)
    while h.size(0) < 16:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    signs = _hash_u32(seed, 0x5EED)
    d = torch.tensor([-1.0 if (signs >> i) & 1 else 1.0 for i in range(16)])
    return (d.view(-1, 1) * h.t() * 0.25).to(device)


def _hash_u32(a: int, b: int) -> int:
    m = 0xFFFFFFFF
    h = ((a * 0x9E3779B1) & m) ^ ((b + 0x7F4A7C15 + ((a << 6) & m) + (a >> 2)) & m)
    h ^= h >> 16
    h = (h * 0x85EBCA6B) & m
    h ^= h >> 13
    h = (h * 0xC2B2AE35) & m
    h ^= h >> 16
    return h


def quantize_nvfp4_reference(x: torch.Tensor, *, two_d: bool = False, hadamard_seed: int = 0, amax: torch.Tensor | None = None,
                             uniforms: torch.Tensor | None = None) -> ScaledOperand:
    rows, K = x.shape
    Kp = -(-K // 16) * 16
    xf = torch.zeros(rows, Kp, dtype=torch.float32, device=x.device)
    xf[:, :K] = x.float()
    if amax is None:
        amax = x.detach().abs().amax().float()
    blocks = xf.view(rows, Kp // 16, 16)
    if hadamard_seed:
        blocks = blocks @ hadamard16(hadamard_seed, x.device)
    bmax = blocks.abs().amax(-1)
    if two_d:
        Rp = -(-rows // 16) * 16
        padded = torch.zeros(Rp, Kp // 16, device=x.device)
        padded[:rows] = bmax
        bmax = padded.view(Rp // 16, 16, -1).amax(1).repeat_interleave(16, 0)[:rows]
    # tensor / tensor: true IEEE divisions, as in the kernel (a Python-scalar operand would multiply by a reciprocal)
    s_enc = torch.where(amax > 0, torch.full_like(amax, NVFP4_RANGE) / amax, torch.ones_like(amax))
    sbyte = (bmax / torch.full_like(bmax, 6.0) * s_enc).clamp(max=448.0).to(torch.float8_e4m3fn)
    sdec = sbyte.float()
    enc = torch.where(sdec > 0, s_enc / sdec, torch.zeros_like(sdec))
    a = blocks * enc.unsqueeze(-1)
    code = _e2m1_encode(a.abs(), None if uniforms is None else uniforms.view(rows, Kp // 16, 16)) | ((a < 0).long() << 3)
    code = code.view(rows, Kp)[:, :K]
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).to(torch.uint8)
    n_sf = Kp // 16
    chunks_k = -(-K // 256) * 4
    sf = torch.zeros(sf_bytes("nvfp4", rows, K), dtype=torch.uint8, device=x.device)
    sf[sf_index(rows, n_sf, chunks_k, x.device).view(-1)] = sbyte.view(torch.uint8).view(-1)
    return ScaledOperand("nvfp4", packed.contiguous(), sf, rows, K, amax=amax)


def decode(op: ScaledOperand) -> torch.Tensor:
    """The fp32 matrix an operand stands for (NVFP4 after the Hadamard transform, if one was applied)."""
    dev = op.data.device
    if op.kind == "fp8":
        dt = torch.float8_e5m2 if op.e5m2 else torch.float8_e4m3fn
        vals = op.data.view(dt).float()
        n_sf = -(-op.K // 32)
        e = op.sf[sf_index(op.rows, n_sf, op.chunks_k, dev)].to(torch.int32) - 127
        scale = torch.ldexp(torch.ones(op.rows, n_sf, device=dev), e).repeat_interleave(32, 1)[:, :op.K]
        return vals * scale
    grid = torch.tensor(E2M1_GRID, device=dev)
    lo, hi = op.data & 0xF, op.data >> 4
    code = torch.stack([lo, hi], -1).view(op.rows, -1).long()
    vals = grid[code & 7] * torch.where((code & 8) > 0, -1.0, 1.0)
    n_sf = -(-op.K // 16)
    sdec = op.sf[sf_index(op.rows, n_sf, op.chunks_k, dev)].view(torch.float8_e4m3fn).float()
    tscale = torch.where(op.amax > 0, op.amax / NVFP4_RANGE, torch.ones_like(op.amax))
    return vals * sdec.repeat_interleave(16, 1)[:, :op.K] * tscale


def reference_gemm(a: ScaledOperand, b: ScaledOperand, alpha: float = 1.0) -> torch.Tensor:
    return alpha * (decode(a).double() @ decode(b).double().t()).float()


# ------------------------------------------------------------------------------------------------
# GPU path
# ------------------------------------------------------------------------------------------------
def _on_gpu(x: torch.Tensor) -> bool:
    return x.is_cuda and native.available()


def quantize_fp8(x: torch.Tensor, block: int = 32, e5m2: bool = False, *, sf_out: torch.Tensor | None = None) -> ScaledOperand:
    """bf16 [rows, K] -> fp8 operand.  block: 32 (MX), 128 (1 x 128) or -128 (128 x 128 blocks)."""
    if block not in (32, 128, -128):
        raise ValueError("block must be 32, 128 or -128")
    rows, K = x.shape
    if not _on_gpu(x):
        return quantize_fp8_reference(x, block, e5m2)
    x = x.contiguous() if x.stride(1) != 1 or x.stride(0) % 4 else x
    if x.dtype != torch.bfloat16:
        x = x.bfloat16()
    q = torch.empty(rows, K, dtype=torch.uint8, device=x.device)
    need = sf_bytes("fp8", rows, K)
    sf = sf_out if sf_out is not None else torch.zeros(need, dtype=torch.uint8, device=x.device)
    rc = native.lib().nga_quant_mxfp8(x.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, K, x.stride(0), q.stride(0), block,
                                      int(e5m2), native.stream_ptr())
    native.check(rc, "nga_quant_mxfp8")
    return ScaledOperand("fp8", q, sf, rows, K, e5m2)


def quantize_nvfp4(x: torch.Tensor, *, two_d: bool = False, hadamard_seed: int = 0, sr_seed: int = 0,
                   amax: torch.Tensor | None = None) -> ScaledOperand:
    rows, K = x.shape
    if amax is None:
        amax = x.detach().abs().amax().float()
    if not _on_gpu(x):
        u = None
        if sr_seed:
            u = torch.rand(rows, -(-K // 16) * 16, generator=torch.Generator().manual_seed(sr_seed))
        return quantize_nvfp4_reference(x, two_d=two_d, hadamard_seed=hadamard_seed, amax=amax, uniforms=u)
    if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.stride(0) % 8:
        x = x.bfloat16().contiguous()
    q = torch.empty(rows, K // 2, dtype=torch.uint8, device=x.device)
    sf = torch.zeros(sf_bytes("nvfp4", rows, K), dtype=torch.uint8, device=x.device)
    amax = amax.reshape(1).contiguous()
    rc = native.lib().nga_quant_nvfp4(x.data_ptr(), q.data_ptr(), sf.data_ptr(), amax.data_ptr(), rows, K, x.stride(0),
                                      q.stride(0), int(two_d), hadamard_seed & 0xFFFFFFFF, sr_seed & 0xFFFFFFFF,
                                      native.stream_ptr())
    native.check(rc, "nga_quant_nvfp4")
    return ScaledOperand("nvfp4", q, sf, rows, K, amax=amax.view(()))


def gemm(a: ScaledOperand, b: ScaledOperand, *, alpha: float = 1.0, out_dtype=torch.bfloat16, epi: int = native.EPI_SCALE,
         aux: torch.Tensor | None = None, beta: float = 0.0) -> torch.Tensor:
    """alpha * a b^T over the shared K (bf16 or fp32 output); NVFP4 tensor scales are applied on the device."""
    if a.kind != b.kind or a.K != b.K:
        raise ValueError("operands differ in format or K")
    M, N, K = a.rows, b.rows, a.K
    if not _on_gpu(a.data):
        out = reference_gemm(a, b, alpha)
        if epi == native.EPI_AXPBY:
            out = out + beta * aux.float()
        elif epi == native.EPI_RELU2:
            out = out.clamp_min(0).square()
        return out.to(out_dtype)
    out = torch.empty(M, N, dtype=out_dtype, device=a.data.device)
    L = native.lib()
    st = native.status_word(a.data.device).data_ptr()
    auxp = None if aux is None else aux.data_ptr()
    ldaux = 0 if aux is None else aux.stride(0)
    aux32 = int(aux is not None and aux.dtype == torch.float32)
    if a.kind == "fp8":
        rc = L.nga_gemm_mxfp8(a.data.data_ptr(), a.sf.data_ptr(), b.data.data_ptr(), b.sf.data_ptr(), out.data_ptr(), auxp, M, N, K,
                              a.data.stride(0), b.data.stride(0), out.stride(0), ldaux, int(a.e5m2), int(b.e5m2), epi,
                              int(out_dtype == torch.float32), aux32, float(alpha), float(beta), st, native.stream_ptr())
    else:
        rc = L.nga_gemm_nvfp4(a.data.data_ptr(), a.sf.data_ptr(), b.data.data_ptr(), b.sf.data_ptr(), out.data_ptr(), auxp, M, N, K,
                              a.data.stride(0), b.data.stride(0), out.stride(0), ldaux, epi, int(out_dtype == torch.float32),
                              aux32, float(alpha), float(beta), a.amax.data_ptr(), b.amax.data_ptr(), st, native.stream_ptr())
    native.check(rc, "nga_gemm_" + ("mxfp8" if a.kind == "fp8" else "nvfp4"))
    return out


def grouped_gemm(a: ScaledOperand, b: ScaledOperand, group_of_mtile: torch.Tensor, groups: int, n_per_group: int, *,
                 alpha: float = 1.0) -> torch.Tensor:
    """Expert form: ``b`` stacks ``groups`` matrices of ``n_per_group`` rows; every 256-row tile of ``a`` multiplies
    the matrix of ``group_of_mtile[tile]`` (int32 device tensor)."""
    M, K = a.rows, a.K
    if b.rows != groups * n_per_group or n_per_group % 128:
        raise ValueError("stacked operand must hold groups x n_per_group rows, n_per_group a multiple of 128")
    if not _on_gpu(a.data):
        da, db = decode(a), decode(b).view(groups, n_per_group, K)
        out = torch.zeros(M, n_per_group)
        for t, g in enumerate(group_of_mtile.tolist()):
            out[t * 256:(t + 1) * 256] = alpha * da[t * 256:(t + 1) * 256] @ db[g].t()
        return out.bfloat16()
    out = torch.empty(M, n_per_group, dtype=torch.bfloat16, device=a.data.device)
    nvf4 = a.kind == "nvfp4"
    rc = native.lib().nga_gemm_grouped_bs(2 if nvf4 else 1, a.data.data_ptr(), a.sf.data_ptr(), b.data.data_ptr(), b.sf.data_ptr(),
                                          out.data_ptr(), group_of_mtile.data_ptr(), groups, M, n_per_group, K, a.data.stride(0),
                                          b.data.stride(0), out.stride(0), float(alpha),
                                          a.amax.data_ptr() if nvf4 else None, b.amax.data_ptr() if nvf4 else None,
                                          native.status_word(a.data.device).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_gemm_grouped_bs")
    return out


# ------------------------------------------------------------------------------------------------
# Linear layer: block-FP8 forward, straight-through backward
# ------------------------------------------------------------------------------------------------
class _BlockFp8Linear(torch.autograd.Function):
    """``y = Q(x) Q(W)^T`` on the block-scaled FP8 GEMM (activations 1 x 128, weights 128 x 128, power-of-two
    scales); the gradients pass straight through the rounding and are taken against the unrounded bf16 operands,
    which is how the reference trains its V4.1 linears (``rounded_activation`` with an identity gradient in front
    of a bf16 linear, src/archlab/architectures/deepseek_v41_torch.py:80-121)."""

    @staticmethod
    def forward(ctx, x, w):
        from . import gemm as G  # noqa: F401  (kernels for the backward)

        x2 = x.reshape(-1, x.size(-1)).to(torch.bfloat16).contiguous()
        wb = w.to(torch.bfloat16)
        ctx.save_for_backward(x2, wb)
        ctx.lead, ctx.dtypes = x.shape[:-1], (x.dtype, w.dtype)
        y = gemm(quantize_fp8(x2, 128), quantize_fp8(wb, -128), out_dtype=torch.bfloat16)
        return y.reshape(*x.shape[:-1], w.size(0)).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        from . import gemm as G

        x2, wb = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1)).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(dy2, wb, b_mn=True, out_dtype=torch.bfloat16).reshape(*ctx.lead, wb.size(1)).to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            dw = G.gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.bfloat16).to(ctx.dtypes[1])
        return dx, dw


def block_fp8_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Bias-free linear with both operands rounded to block-scaled FP8 in the forward product."""
    return _BlockFp8Linear.apply(x, weight)


def block_fp8_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return _on_gpu(x) and weight.size(1) % 128 == 0 and weight.size(0) % 8 == 0 and x.size(-1) == weight.size(1)


# ------------------------------------------------------------------------------------------------
# Linear layer: NVFP4 training (forward, data gradient and weight gradient all on the FP4 tensor-core path)
# ------------------------------------------------------------------------------------------------
NVFP4_ALIGNMENT = 128          # both sides of a dense weight: keeps the reduction of all three GEMMs Hadamard-tile aligned


class _Nvfp4Linear(torch.autograd.Function):
    """The controls of the reference's NVFP4 recipe (src/archlab/speedrun/precision.py:170-205): weights in 16 x 16
    blocks (so the transposed weight carries the same scales), stochastic rounding on gradients, a random Hadamard
    transform on both operands of the weight-gradient product (it cancels in the product and spreads outliers).
    Every product is ``A B^T`` with K contiguous, so the backward quantises transposed copies."""

    @staticmethod
    def forward(ctx, x, w, seed):
        x2 = x.reshape(-1, x.size(-1)).to(torch.bfloat16).contiguous()
        wb = w.to(torch.bfloat16).contiguous()
        ctx.save_for_backward(x2, wb)
        ctx.lead, ctx.dtypes, ctx.seed = x.shape[:-1], (x.dtype, w.dtype), int(seed)
        y = gemm(quantize_nvfp4(x2), quantize_nvfp4(wb, two_d=True), out_dtype=torch.bfloat16)
        return y.reshape(*x.shape[:-1], w.size(0)).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x2, wb = ctx.saved_tensors
        seed = ctx.seed
        dy2 = dy.reshape(-1, dy.size(-1)).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dX [M, K] = dY [M, N] W [N, K]: reduction over N -> B operand is W^T [K, N]
            dx = gemm(quantize_nvfp4(dy2, sr_seed=seed), quantize_nvfp4(wb.t().contiguous(), two_d=True), out_dtype=torch.bfloat16)
            dx = dx.reshape(*ctx.lead, wb.size(1)).to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            # dW [N, K] = dY^T [N, M] X^T[K, M]^T: reduction over the tokens, both operands Hadamard-transformed along it
            M = dy2.size(0)
            pad = (-M) % 16
            dyt, xt = dy2.t().contiguous(), x2.t().contiguous()
            if pad:
                dyt, xt = torch.nn.functional.pad(dyt, (0, pad)), torch.nn.functional.pad(xt, (0, pad))
            dw = gemm(quantize_nvfp4(dyt, hadamard_seed=seed | 1, sr_seed=seed + 1),
                      quantize_nvfp4(xt, hadamard_seed=seed | 1), out_dtype=torch.float32).to(ctx.dtypes[1])
        return dx, dw, None


def nvfp4_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (weight.size(0) % NVFP4_ALIGNMENT == 0 and weight.size(1) % NVFP4_ALIGNMENT == 0 and x.size(-1) == weight.size(1)
            and x.numel() // x.size(-1) % 64 == 0)


def nvfp4_linear(x: torch.Tensor, weight: torch.Tensor, seed: int = 1) -> torch.Tensor:
    """Bias-free linear whose three products run in NVFP4; ``seed`` drives stochastic rounding and the Hadamard signs
    (pass the step number for fresh rounding noise every step)."""
    return _Nvfp4Linear.apply(x, weight, seed)


class BlockScaledLinear(torch.nn.Linear):
    """``nn.Linear`` (no bias) re-classed onto a block-scaled recipe: ``recipe`` is "nvfp4" or "fp8_block".  Shapes the
    recipe does not cover (a side not divisible by 128, a ragged token count) run in bf16 on the tcgen05 kernels -
    the BF16 exceptions of the reference's FP4 contract (src/archlab/architectures/qwen38_flash_next.py:160-175)."""

    recipe = "nvfp4"
    step = 0

    def forward(self, x):
        w = self.weight
        if self.recipe == "nvfp4" and nvfp4_supported(x, w):
            return nvfp4_linear(x, w, seed=2 * self.step + 1)
        if self.recipe == "fp8_block" and (block_fp8_supported(x, w) or not x.is_cuda) and w.size(1) % 128 == 0:
            return block_fp8_linear(x, w)
        from .native_linear import native_linear

        return native_linear(x, w)


def convert_linears(module: torch.nn.Module, recipe: str, *, skip: tuple[str, ...] = ("lm_head", "router", "gate")) -> dict:
    """Re-classes the eligible bias-free linears of ``module`` in place and reports what ran where:
    ``{"converted": [...], "bf16_exceptions": {name: reason}}``.  Routing logits, scalar gates and the output head stay
    in bf16 by name; a weight side not divisible by 128 stays in bf16 by shape."""
    if recipe not in ("nvfp4", "fp8_block"):
        raise ValueError("recipe must be 'nvfp4' or 'fp8_block'")
    report = {"recipe": recipe, "converted": [], "bf16_exceptions": {}}
    for name, layer in module.named_modules():
        if type(layer) is not torch.nn.Linear and type(layer).__name__ != "CastLinear":
            continue
        if layer.bias is not None:
            report["bf16_exceptions"][name] = "bias"
        elif any(part in name.split(".")[-1] for part in skip):
            report["bf16_exceptions"][name] = "kept in bf16 by role"
        elif layer.in_features % NVFP4_ALIGNMENT or layer.out_features % NVFP4_ALIGNMENT:
            report["bf16_exceptions"][name] = f"{layer.out_features} x {layer.in_features} is not 128-aligned"
        else:
            layer.__class__ = type("BlockScaledLinear_" + recipe, (BlockScaledLinear,), {"recipe": recipe})
            report["converted"].append(name)
    return report


def set_step(module: torch.nn.Module, step: int) -> None:
    """Advances the rounding-noise seed of every converted layer (call once per optimizer step)."""
    for layer in module.modules():
        if isinstance(layer, BlockScaledLinear):
            layer.step = step
