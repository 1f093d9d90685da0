"""bf16 GEMM with fused epilogues on the tcgen05 kernel (``csrc/gemm.cu``).

``gemm(a, b, a_mn=…, b_mn=…)`` computes ``D = epi(alpha * A @ B^T, aux)`` where the logical A is
``M x K`` and the logical B is ``N x K``:

* ``a_mn=False``: ``a`` is stored ``[M, K]`` (K contiguous); ``a_mn=True``: stored ``[K, M]``.
* ``b_mn=False``: ``b`` is stored ``[N, K]``; ``b_mn=True``: stored ``[K, N]``.

So a linear layer ``y = x W^T`` uses ``gemm(x, W)``, its dgrad ``gemm(dy, W, b_mn=True)`` and its
wgrad ``gemm(dy, x, a_mn=True, b_mn=True)``, none of which needs a transposed copy.  A leading
batch dimension is supported on all operands.  CPU tensors take an fp32 PyTorch path (that path
is the numerical oracle of the GPU tests); CUDA tensors always run the native kernel.
"""
from __future__ import annotations

import os

import torch

from . import native

__all__ = ["gemm", "EPI_SCALE", "EPI_AXPBY", "EPI_RELU2", "EPI_MUL_DRELU2", "EPI_ATOMIC_ADD"]

# EPI_ATOMIC_ADD: out (fp32, must already hold valid data) += alpha * A @ B^T through vector atomics;
# the contraction may then be split over K (``splits``) so that few-tile / long-K problems such as
# weight gradients still fill the machine.
EPI_SCALE, EPI_AXPBY, EPI_RELU2, EPI_MUL_DRELU2, EPI_ATOMIC_ADD = 0, 1, 2, 3, 4

# "auto": CTA-pair kernel (cta_group::2, 256 x 256 tiles) when the problem has enough such tiles to
# fill the machine, otherwise the single-CTA 128 x {128, 256} kernel.  "single" / "pair" force one.
DEFAULT_IMPL = os.environ.get("NGA_GEMM_IMPL", "auto")


def _logical(a: torch.Tensor, mn: bool) -> torch.Tensor:
    return a.transpose(-1, -2) if mn else a


def gemm_reference(a, b, *, a_mn=False, b_mn=False, aux=None, epi=EPI_SCALE, alpha=1.0, beta=0.0,
                   out_dtype=torch.bfloat16):
    """fp32 PyTorch statement of the kernel's arithmetic."""
    A = _logical(a, a_mn).float()
    B = _logical(b, b_mn).float()
    acc = alpha * (A @ B.transpose(-1, -2))
    if epi == EPI_SCALE:
        d = acc
    elif epi == EPI_AXPBY:
        d = acc + beta * aux.float()
    elif epi == EPI_RELU2:
        d = torch.relu(acc).square()
    elif epi == EPI_MUL_DRELU2:
        d = acc * 2.0 * aux.float().clamp_min(0).sqrt()
    elif epi == EPI_ATOMIC_ADD:
        d = acc + aux.float()
    else:
        raise ValueError(f"unknown epilogue {epi}")
    return d.to(out_dtype)


def _choose_splits(M: int, N: int, K: int, batch: int, slots: int = 74) -> int:
    """Split-K factor for an atomically accumulated GEMM from a two-term cost model fitted on B200:
    tensor time = (time of one full-K 256 x 256 tile on a CTA pair) * waves / splits, plus one fp32
    reduction pass over the output per split at ~1.3 TB/s of L2 atomic throughput."""
    tiles = ((M + 255) // 256) * ((N + 255) // 256) * batch
    t_tile = 2.0 * 256 * 256 * K / 19.6e12
    t_red = 4.0 * M * N * batch / 1.3e12
    best, best_cost = 1, float("inf")
    for s in range(1, 17):
        if s > 1 and (K // 64) // s < 16:
            break
        cost = t_tile * (-(-tiles * s // slots)) / s + t_red * s
        if cost < best_cost * (1 - 1e-6):
            best, best_cost = s, cost
    return best


def _strides(t: torch.Tensor) -> tuple[int, int, int]:
    """(batch, row stride, batch stride) of a 2-D / 3-D tensor with unit inner stride."""
    if t.stride(-1) != 1:
        raise ValueError("innermost dimension must be contiguous")
    if t.dim() == 2:
        return 1, t.stride(0), 0
    if t.dim() == 3:
        return t.size(0), t.stride(1), t.stride(0)
    raise ValueError("expected a 2-D or 3-D tensor")


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, aux: torch.Tensor | None = None, epi: int = EPI_SCALE,
         alpha: float = 1.0, beta: float = 0.0, out_dtype: torch.dtype = torch.bfloat16,
         impl: str | None = None, splits: int = 0) -> torch.Tensor:
    if a.device.type != "cuda":
        if epi == EPI_ATOMIC_ADD:
            aux = out
        d = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, aux=aux, epi=epi, alpha=alpha, beta=beta,
                           out_dtype=out.dtype if out is not None else out_dtype)
        if out is not None:
            out.copy_(d)
            return out
        return d
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm operands must be bf16")
    ba, lda, sa = _strides(a)
    bb, ldb, sb = _strides(b)
    K = a.size(-2) if a_mn else a.size(-1)
    M = a.size(-1) if a_mn else a.size(-2)
    Kb = b.size(-2) if b_mn else b.size(-1)
    N = b.size(-1) if b_mn else b.size(-2)
    if K != Kb:
        raise ValueError(f"K mismatch: {K} vs {Kb}")
    batch = max(ba, bb)
    if ba != bb:
        raise ValueError("batch mismatch (operands do not broadcast over the batch dimension)")
    if out is None:
        if epi == EPI_ATOMIC_ADD:
            raise ValueError("EPI_ATOMIC_ADD accumulates into an existing output")
        shape = (batch, M, N) if (a.dim() == 3 or b.dim() == 3) else (M, N)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    bo, ldd, sd = _strides(out)
    if out.size(-2) != M or out.size(-1) != N or bo != (batch if out.dim() == 3 else 1):
        raise ValueError("output shape mismatch")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("output must be bf16 or fp32")
    ldaux = saux = 0
    aux_fp32 = 0
    if epi in (EPI_AXPBY, EPI_MUL_DRELU2):
        if aux is None:
            raise ValueError("this epilogue needs aux")
        _, ldaux, saux = _strides(aux)
        if aux.dtype not in (torch.bfloat16, torch.float32):
            raise TypeError("aux must be bf16 or fp32")
        aux_fp32 = int(aux.dtype == torch.float32)
    impl = impl or DEFAULT_IMPL
    tiles_pair = ((M + 255) // 256) * ((N + 255) // 256) * batch
    if epi == EPI_ATOMIC_ADD:
        if out.dtype != torch.float32:
            raise TypeError("EPI_ATOMIC_ADD needs an fp32 output")
        if splits <= 0:
            splits = _choose_splits(M, N, K, batch)
    else:
        splits = 1
    use_pair = impl == "pair" or (impl == "auto" and M >= 256 and N >= 256 and tiles_pair * splits >= 64)
    fn = native.lib().nga_gemm2_bf16 if use_pair else native.lib().nga_gemm_bf16
    rc = fn(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), aux.data_ptr() if aux is not None else None,
        M, N, K, batch, lda, ldb, ldd, ldaux, sa if ba > 1 else 0, sb if bb > 1 else 0, sd, saux,
        int(a_mn), int(b_mn), epi, int(out.dtype == torch.float32), aux_fp32, float(alpha),
        float(beta), int(splits), native.status_word(a.device).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_gemm_bf16")
    return out
