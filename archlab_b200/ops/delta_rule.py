"""Delta-rule linear-attention recurrences: gated delta net (GDN) and Kimi delta attention (KDA).

State ``S_t`` is a ``[key_dim, value_dim]`` matrix per (batch, head):

    S_t = decay_t * S_{t-1} ;  S_t += k_t (beta_t (v_t - k_t^T S_t))^T ;  o_t = S_t^T q_t

GDN uses one scalar log-decay per (token, head); KDA one per key channel.  q and k are L2
normalised, q additionally scaled by ``1/sqrt(K)``.  The O(T) recurrent functions are the oracles
(src/archlab/architectures/qwen38_flash_next_full.py:535-554, kimi.py:154-178; the reference's
kernels are fla-core Triton ``chunk_gated_delta_rule`` / ``chunk_kda``).  ``chunk_*`` are the
chunk-parallel forms (chunk 64: intra-chunk triangular solve + inter-chunk state passing) that the
sm_100a kernels follow; they are differentiable and serve as the CPU / fallback path.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _prep(q, k, v, g, beta):
    K = q.size(-1)
    q = F.normalize(q.float(), p=2, dim=-1) * K ** -0.5
    k = F.normalize(k.float(), p=2, dim=-1)
    return q, k, v.float(), g.float(), beta.float()


def gated_delta_reference(q, k, v, decay, beta):
    """[B, T, H, K] q/k, [B, T, H, V] v, [B, T, H] log-decay (<= 0) and beta -> [B, T, H, V]."""
    q, k, v, decay, beta = _prep(q, k, v, decay, beta)
    B, T, H, K = q.shape
    state = q.new_zeros(B, H, K, v.size(-1))
    outs = []
    for t in range(T):
        state = state * decay[:, t].exp()[..., None, None]
        pred = torch.einsum("bhk,bhkv->bhv", k[:, t], state)
        upd = beta[:, t, :, None] * (v[:, t] - pred)
        state = state + k[:, t, :, :, None] * upd[:, :, None, :]
        outs.append(torch.einsum("bhkv,bhk->bhv", state, q[:, t]))
    return torch.stack(outs, dim=1)


def kda_recurrent_reference(q, k, v, g, beta):
    """As above with a per-channel log-decay ``g`` of shape [B, T, H, K]."""
    q, k, v, g, beta = _prep(q, k, v, g, beta)
    B, T, H, K = q.shape
    state = q.new_zeros(B, H, K, v.size(-1))
    outs = []
    for t in range(T):
        state = state * g[:, t].exp()[..., None]
        pred = torch.einsum("bhk,bhkv->bhv", k[:, t], state)
        upd = beta[:, t, :, None] * (v[:, t] - pred)
        state = state + k[:, t, :, :, None] * upd[:, :, None, :]
        outs.append(torch.einsum("bhkv,bhk->bhv", state, q[:, t]))
    return torch.stack(outs, dim=1)


def _decayed_gram(a: torch.Tensor, b: torch.Tensor, G: torch.Tensor, sub: int = 16) -> torch.Tensor:
    """M[t, s] = sum_c a[t, c] b[s, c] exp(G[t, c] - G[s, c]) for s <= t, else 0, over the last two dims
    ``[C, K]``.  Every exponent that is evaluated is <= 0 (G is non-increasing in t): blocks below the
    diagonal factor through the cumulative decay at the first row of the row block, diagonal
    ``sub x sub`` blocks are evaluated pairwise."""
    C = a.size(-2)
    out = a.new_zeros(*a.shape[:-2], C, C)
    for i0 in range(0, C, sub):
        i1 = min(C, i0 + sub)
        ref = G[..., i0:i0 + 1, :]
        left = a[..., i0:i1, :] * (G[..., i0:i1, :] - ref).exp()
        if i0:
            right = b[..., :i0, :] * (ref - G[..., :i0, :]).clamp_max(0).exp()
            out[..., i0:i1, :i0] = left @ right.transpose(-1, -2)
        diff = (G[..., i0:i1, None, :] - G[..., None, i0:i1, :]).clamp_max(0).exp()       # [sub, sub, K]
        blk = torch.einsum("...tc,...sc,...tsc->...ts", a[..., i0:i1, :], b[..., i0:i1, :], diff)
        out[..., i0:i1, i0:i1] = torch.tril(blk)
    return out


def chunk_kda(q, k, v, g, beta, chunk: int = 64, initial_state=None, output_final_state: bool = False):
    """Chunk-parallel KDA (per-channel decay); GDN is the special case of a channel-constant ``g``.

    Within a chunk with cumulative log-decay ``G_t = sum_{s<=t} g_s`` (per channel) the corrected
    values ``u`` solve the unit-lower-triangular system
        (I + strict_tril(diag(beta) P)) u = beta * (v - (k exp(G)) S_0),  P[t,s] = sum_c k_t k_s exp(G_t - G_s)
    and  o = (q exp(G)) S_0 + tril(Q) u  with Q[t,s] = sum_c q_t k_s exp(G_t - G_s),
         S_C = exp(G_C) * S_0 + (k exp(G_C - G))^T u.
    All exponentials are of non-positive numbers, so strong decays cannot overflow."""
    q, k, v, g, beta = _prep(q, k, v, g, beta)
    B, T, H, K = q.shape
    V = v.size(-1)
    pad = (-T) % chunk
    if pad:
        q, k, v, g = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v, g))
        beta = F.pad(beta, (0, 0, 0, pad))
    n = (T + pad) // chunk
    rs = lambda x: x.view(B, n, chunk, H, -1).permute(0, 1, 3, 2, 4)      # [B, n, H, C, *]
    q, k, v, g = rs(q), rs(k), rs(v), rs(g)
    beta = beta.view(B, n, chunk, H).permute(0, 1, 3, 2)                  # [B, n, H, C]
    G = g.cumsum(dim=-2)
    kd, qd = k * G.exp(), q * G.exp()
    eye = torch.eye(chunk, device=q.device, dtype=q.dtype)
    A = torch.tril(beta[..., None] * _decayed_gram(k, k, G), -1) + eye
    Aq = _decayed_gram(q, k, G)
    Gend = G[..., -1:, :]
    kend = k * (Gend - G).exp()                                            # k_s exp(G_C - G_s)
    state = q.new_zeros(B, H, K, V) if initial_state is None else initial_state.float()
    outs = []
    for c in range(n):
        rhs = beta[:, c, ..., None] * (v[:, c] - kd[:, c] @ state)
        u = torch.linalg.solve_triangular(A[:, c], rhs, upper=False, unitriangular=True)
        outs.append(qd[:, c] @ state + Aq[:, c] @ u)
        state = Gend[:, c].transpose(-1, -2).exp() * state + kend[:, c].transpose(-1, -2) @ u
    o = torch.stack(outs, dim=1).permute(0, 1, 3, 2, 4).reshape(B, n * chunk, H, V)[:, :T]
    return (o, state) if output_final_state else o


def chunk_gated_delta_rule(q, k, v, decay, beta, chunk: int = 64, **kw):
    """GDN: scalar log-decay per (token, head) broadcast over the key channels."""
    return chunk_kda(q, k, v, decay[..., None].expand(*decay.shape, q.size(-1)), beta, chunk, **kw)


def fused_kda_gate(raw_gate: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor | None = None):
    """Per-channel log-decay ``g = -exp(A_log) * softplus(raw + dt_bias)`` (<= 0); ``a_log`` is per head."""
    x = raw_gate.float()
    if dt_bias is not None:
        x = x + dt_bias.float().view(*([1] * (x.dim() - 2)), *x.shape[-2:]) if dt_bias.dim() == 2 else x + dt_bias.float()
    return -a_log.float().exp().view(*([1] * (x.dim() - 2)), -1, 1) * F.softplus(x)


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                  activation: str | None = "silu", dilation: int = 1) -> torch.Tensor:
    """Depthwise causal convolution over [B, T, C] with weight [C, k] (k = 4 in every reference
    model; src/archlab/architectures/qwen38_flash_next_full.py:491-532), optional SiLU."""
    B, T, Cc = x.shape
    kk = weight.size(1)
    y = F.conv1d(F.pad(x.transpose(1, 2), ((kk - 1) * dilation, 0)), weight.unsqueeze(1).to(x.dtype), bias,
                 groups=Cc, dilation=dilation).transpose(1, 2)
    if activation == "silu":
        y = F.silu(y)
    elif activation is not None:
        raise ValueError(f"unsupported activation {activation!r}")
    return y


# ------------------------------------------------------------------------------------------------
# sm_100a kernel path (gated delta rule, scalar decay, width 128)
# ------------------------------------------------------------------------------------------------
def _native():
    import ctypes as C

    from . import native

    vp, i = C.c_void_p, C.c_int
    native.register_signature("nga_gdn_workspace_bytes", [i, i, i], C.c_longlong)
    native.register_signature("nga_gdn_fwd", [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, vp, vp])
    return native


def gdn_kernel_supports(q, k, v) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.size(-1) == 128 and v.size(-1) == 128 and k.shape == q.shape
            and v.shape[:3] == q.shape[:3])


def gdn_forward_cuda(q, k, v, decay, beta, initial_state=None, output_final_state: bool = False):
    """Forward of the gated delta rule on the tcgen05 kernels: q/k/v [B, T, H, 128] bf16 (un-normalised),
    decay/beta [B, T, H].  Returns o [B, T, H, 128] bf16 (and the final fp32 state [B, H, 128, 128])."""
    native = _native()
    B, T, H, D = q.shape
    pad = (-T) % 64
    if pad:                                              # zero k, v, beta and zero log-decay leave the state untouched
        q, k, v = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v))
        decay, beta = F.pad(decay, (0, 0, 0, pad)), F.pad(beta, (0, 0, 0, pad))
    Tp = T + pad
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    g32, b32 = decay.float().contiguous(), beta.float().contiguous()
    o = torch.empty(B, Tp, H, D, dtype=torch.bfloat16, device=q.device)
    ws = torch.empty(native.lib().nga_gdn_workspace_bytes(B, Tp, H), dtype=torch.uint8, device=q.device)
    s0 = None if initial_state is None else initial_state.float().contiguous()
    s_out = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device) if output_final_state else None
    ptr = lambda t: None if t is None else t.data_ptr()
    rc = native.lib().nga_gdn_fwd(ptr(q), ptr(k), ptr(v), ptr(g32), ptr(b32), ptr(o), ptr(s0), ptr(s_out), ptr(ws), B, Tp, H, D,
                                  native.status_word(q.device).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_gdn_fwd")
    o = o[:, :T]
    return (o, s_out) if output_final_state else o


class _GatedDeltaFn(torch.autograd.Function):
    """Kernel forward; the backward differentiates the chunk-parallel PyTorch form on the saved inputs."""

    @staticmethod
    def forward(ctx, q, k, v, decay, beta):
        ctx.save_for_backward(q, k, v, decay, beta)
        return gdn_forward_cuda(q, k, v, decay, beta)

    @staticmethod
    def backward(ctx, do):
        saved = [t.detach().requires_grad_(True) for t in ctx.saved_tensors]
        with torch.enable_grad():
            o = chunk_gated_delta_rule(*saved)
        grads = torch.autograd.grad(o, saved, do.float())
        return tuple(g.to(t.dtype) for g, t in zip(grads, ctx.saved_tensors))


def gated_delta_rule(q, k, v, decay, beta):
    """Dispatch: tcgen05 forward for bf16 CUDA inputs of width 128, else the chunk-parallel PyTorch form."""
    if gdn_kernel_supports(q, k, v):
        return _GatedDeltaFn.apply(q, k, v, decay, beta)
    return chunk_gated_delta_rule(q, k, v, decay, beta).to(q.dtype)
