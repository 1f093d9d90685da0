"""DeepSeek-V4.1-style sparse-MoE language model.

Per layer: 4-stream hyper-connection residual (coefficients from ``hc_split_sinkhorn``), DSA sparse
attention (lightning indexer -> top-k keys -> gathered MQA over a shared latent KV with a sink
logit), and a MoE feed-forward (routed experts with a sqrt-softplus / sigmoid router, aux-free
selection bias, shared experts, clamped SwiGLU).  Linear layers optionally train through block-
scaled FP8 rounding (activations 1 x 128, weights 128 x 128, straight-through gradients).

Reference pieces: src/archlab/architectures/deepseek_v41_adapter.py:23-152,
deepseek_v41_torch.py:16-121, deepseek_v41_math.py:14-62, deepseek_v41_inference_moe.py:9-47,
dsa.py:20-429; expert parallelism src/archlab/automodel/deepseek_v41_parallel.py:16-111.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import blockscaled, dsa, dsa_cuda, quant, stream_mix
from . import moe
from .blocks import RMSNorm, apply_rope, hc_split_sinkhorn, rms_norm, rope_tables


@dataclass(frozen=True)
class V41Config:
    vocab_size: int = 129_280
    sequence_len: int = 4096
    n_layer: int = 24
    hidden_size: int = 2048
    n_heads: int = 16
    head_dim: int = 128
    rope_dim: int = 64
    rope_theta: float = 10000.0
    index_heads: int = 4
    index_head_dim: int = 64
    index_rope_dim: int = 32
    index_top_k: int = 2048
    dense_warmup_steps: int = 0
    indexer_kl_weight: float = 1.0
    indexer_kl_rows: int = 512            # query rows per sequence on which the KL target is evaluated (0: all)
    n_routed_experts: int = 64
    n_shared_experts: int = 2
    experts_top_k: int = 6
    moe_inter: int = 1408
    router_score: str = "sigmoid"
    route_scale: float = 1.0
    swiglu_limit: float | None = 7.0
    hc_streams: int = 4
    hc_sinkhorn_iters: int = 20
    fp8: bool = False
    fp8_block: int = 128
    # expert-parallel layers over peer memory.  None: the exact segment sizes are read back per layer (one host
    # synchronisation each, always correct).  A factor f or "auto": grouped GEMMs run over a fixed bound of rows (f x tokens
    # x top-k, or 1.5 x the largest row count of the previous step) whose layout lives on the device, with no host
    # synchronisation; a step that exceeds the bound raises at its end.  The untrained router of the 24-layer model moved
    # its load by more than 1.5x between early steps, so the exact form is the default and the bound is a tuning choice
    # (2.8 % of the step on a 6-layer slice).
    expert_capacity_factor: float | str | None = None
    rms_eps: float = 1e-6

    @classmethod
    def tiny(cls, **kw) -> "V41Config":
        base = dict(vocab_size=256, sequence_len=64, n_layer=2, hidden_size=64, n_heads=4, head_dim=16, rope_dim=8,
                    index_heads=2, index_head_dim=16, index_rope_dim=8, index_top_k=8, n_routed_experts=8,
                    n_shared_experts=1, experts_top_k=2, moe_inter=32, fp8_block=32)
        base.update(kw)
        return cls(**base)

    def to_dict(self):
        return asdict(self)


class QuantLinear(nn.Linear):
    """``y = x W^T`` with optional block-FP8 rounding of both operands (straight-through)."""

    def __init__(self, i, o, *, fp8=False, block=128):
        super().__init__(i, o, bias=False)
        self.fp8, self.block = fp8, block

    def forward(self, x):
        if not self.fp8 or x.size(-1) % self.block:
            return moe.dense_linear(x, self.weight)                  # tcgen05 kernels on a GPU, F.linear otherwise
        if self.block == 128 and blockscaled.block_fp8_supported(x, self.weight):
            return blockscaled.block_fp8_linear(x, self.weight)      # the product itself runs in FP8 on the tensor core
        xq = quant.rounded_activation(x, bits=8, block_size=self.block)
        with torch.no_grad():
            wq, ws = quant.fp8_weight_quantize_2d(self.weight, self.block)
            wr = quant.fp8_weight_dequantize_2d(wq, ws, self.block).to(self.weight.dtype)
        w = self.weight + (wr - self.weight).detach()
        return F.linear(xq, w.to(x.dtype))


class LightningIndexer(nn.Module):
    def __init__(self, c: V41Config):
        super().__init__()
        self.h, self.d, self.rope, self.top_k = c.index_heads, c.index_head_dim, c.index_rope_dim, c.index_top_k
        self.q_proj = nn.Linear(c.hidden_size, self.h * self.d, bias=False)
        self.k_proj = nn.Linear(c.hidden_size, self.d, bias=False)
        self.k_norm = nn.LayerNorm(self.d, eps=1e-6)
        self.weights_proj = nn.Linear(c.hidden_size, self.h, bias=False)

    def forward(self, x: torch.Tensor, cos, sin, fused: bool = False):
        """-> (scores [B,S,S] fp32 causal, indices [B,S,k] with -1 padding), or (None, None) with ``self.bits`` set
        when ``fused`` and the selection kernel applies.  Inputs are detached: the indexer learns only from its
        KL objective."""
        x = x.detach()
        B, S, _ = x.shape
        q = self.q_proj(x).view(B, S, self.h, self.d)
        k = self.k_norm(self.k_proj(x).float()).to(x.dtype).unsqueeze(2)
        q = apply_rope(q, cos, sin, rot_dim=self.rope)
        k = apply_rope(k, cos, sin, rot_dim=self.rope).squeeze(2)
        w = self.weights_proj(x).float() * self.h ** -0.5
        self.qkw = (q, k, w)                               # for the objective on a subset of rows
        if fused and dsa_cuda.indexer_kernel_supports(q, k):
            # selection kernel: scores, top-k threshold and one bit per key without the [S, S] score matrix
            self.bits = dsa_cuda.indexer_select(q, k, w, self.top_k) if S > self.top_k else None
            return None, None
        self.bits = None
        scores = dsa.indexer_scores(q, k, w)
        idx, vals = dsa.select_topk(scores, self.top_k)
        self.kth = vals[..., -1:].detach()                 # threshold form of the same selection (for the bit-mask kernels)
        return scores, idx

    def scores_for_rows(self, rows: torch.Tensor) -> torch.Tensor:
        """Differentiable scores of the given query rows against all keys (the rows the objective looks at)."""
        q, k, w = self.qkw
        return dsa.indexer_scores(q[:, rows], k, w[:, rows], positions=rows)


class SparseLatentAttention(nn.Module):
    """Multi-query attention over one shared latent KV vector per token (key = value), restricted to
    the indexer's top-k keys, with a learned per-head sink."""

    def __init__(self, c: V41Config):
        super().__init__()
        self.c = c
        self.h, self.d = c.n_heads, c.head_dim
        mk = lambda i, o: QuantLinear(i, o, fp8=c.fp8, block=c.fp8_block)
        self.q_proj = mk(c.hidden_size, self.h * self.d)
        self.kv_proj = mk(c.hidden_size, self.d)
        self.q_norm = RMSNorm(self.d, c.rms_eps)
        self.kv_norm = RMSNorm(self.d, c.rms_eps)
        self.sink = nn.Parameter(torch.zeros(self.h))
        self.o_proj = mk(self.h * self.d, c.hidden_size)
        self.indexer = LightningIndexer(c)
        self.last_kl = None
        self.kl_step = 0

    def forward(self, x, cos, sin, *, dense: bool = False):
        B, S, _ = x.shape
        q = apply_rope(self.q_norm(self.q_proj(x).view(B, S, self.h, self.d)), cos, sin, rot_dim=self.c.rope_dim)
        kv = apply_rope(self.kv_norm(self.kv_proj(x)).unsqueeze(2), cos, sin, rot_dim=self.c.rope_dim).squeeze(2)
        scale = self.d ** -0.5
        icos, isin = cos[:, : self.c.index_rope_dim // 2], sin[:, : self.c.index_rope_dim // 2]
        flash = dsa_cuda.kernel_supports(q, kv)
        scores, idx = self.indexer(x, icos, isin, fused=flash)
        if self.training and self.c.indexer_kl_weight > 0:
            rows = dsa.kl_rows(S, self.c.indexer_kl_rows, self.kl_step, x.device)
            self.kl_step += 1
            if rows is None and scores is None:
                rows = torch.arange(S, device=x.device)
            if rows is None:
                target = dsa.main_attention_target(q, kv, scale)
                self.last_kl = dsa.indexer_kl(target, scores, torch.isfinite(scores))
            else:                                        # the [heads, S, S] target is the costliest tensor of the layer
                target = dsa.main_attention_target(q[:, rows], kv, scale, rows)
                sub = scores[:, rows] if scores is not None else self.indexer.scores_for_rows(rows)
                self.last_kl = dsa.indexer_kl(target, sub, torch.isfinite(sub))
        use_dense = dense or S <= self.c.index_top_k
        if flash:                                            # flash kernels with selection bits and sink
            if use_dense:
                o = dsa_cuda.selected_sink_attention(q, kv, self.sink)
            elif scores is None:
                o = dsa_cuda.selected_sink_attention(q, kv, self.sink, bits_pair=self.indexer.bits)
            else:
                o = dsa_cuda.selected_sink_attention(q, kv, self.sink, scores=scores.detach(), kth=self.indexer.kth)
        elif use_dense:
            o = dsa.dense_sink_attention(q, kv, self.sink, scale)
        else:
            o = dsa.sparse_attention(q, kv, self.sink, idx, scale)
        return self.o_proj(o.reshape(B, S, self.h * self.d).to(x.dtype))


class HyperConnectionMix(nn.Module):
    """V4.1 n-stream residual: project the normalised packed streams to ``(n + 2) n`` mixing logits;
    pre-weights collapse the streams into the sublayer input, post-weights write the output back,
    the Sinkhorn-balanced ``comb`` matrix mixes the residual streams."""

    def __init__(self, c: V41Config):
        super().__init__()
        self.n, self.iters, self.eps = c.hc_streams, c.hc_sinkhorn_iters, c.rms_eps
        n = self.n
        self.proj = nn.Linear(n * c.hidden_size, (n + 2) * n, bias=False)
        self.scale = nn.Parameter(torch.full((3,), 0.01))
        base = torch.zeros((n + 2) * n)
        base[2 * n:] = (torch.eye(n) * 4.0).flatten()         # start close to the identity mixing
        self.base = nn.Parameter(base)

    def coefficients(self, streams: torch.Tensor):
        flat = rms_norm(streams.flatten(-2).float(), eps=self.eps)
        return hc_split_sinkhorn(F.linear(flat, self.proj.weight.float()), self.scale, self.base, self.n, self.iters)

    def forward(self, streams: torch.Tensor, sublayer):
        pre, post, comb = self.coefficients(streams)
        x = stream_mix.hyper_connection_read(pre, streams)       # one fused pass on bf16 CUDA, einsum elsewhere
        y = sublayer(x)
        return stream_mix.hyper_connection_write(comb, post, streams, y.to(streams.dtype))


class V41Block(nn.Module):
    def __init__(self, c: V41Config, ep_group=None, ep_buffers=None):
        super().__init__()
        self.attn_norm, self.ffn_norm = RMSNorm(c.hidden_size, c.rms_eps), RMSNorm(c.hidden_size, c.rms_eps)
        self.attn = SparseLatentAttention(c)
        if ep_buffers is not None:                      # dispatch / combine kernels over peer memory
            from ..parallel.ep import FusedExpertParallelMoE

            self.ffn = FusedExpertParallelMoE(c.hidden_size, c.moe_inter, c.n_routed_experts, c.experts_top_k, ep_buffers,
                                              score=c.router_score, route_scale=c.route_scale, swiglu_limit=c.swiglu_limit,
                                              n_shared=c.n_shared_experts, fp8=c.fp8 and c.fp8_block == 128,
                                              capacity_factor=c.expert_capacity_factor)
        elif ep_group is not None:
            self.ffn = moe.ExpertParallelMoE(c.hidden_size, c.moe_inter, c.n_routed_experts, c.experts_top_k, ep_group,
                                             score=c.router_score, route_scale=c.route_scale, swiglu_limit=c.swiglu_limit,
                                             n_shared=c.n_shared_experts)
        else:
            self.ffn = moe.SparseMoE(c.hidden_size, c.moe_inter, c.n_routed_experts, c.experts_top_k,
                                     n_shared=c.n_shared_experts, score=c.router_score, route_scale=c.route_scale,
                                     swiglu_limit=c.swiglu_limit)
        self.hc_attn, self.hc_ffn = HyperConnectionMix(c), HyperConnectionMix(c)

    def forward(self, streams, cos, sin, dense: bool):
        streams = self.hc_attn(streams, lambda x: self.attn(self.attn_norm(x), cos, sin, dense=dense))
        return self.hc_ffn(streams, lambda x: self.ffn(self.ffn_norm(x)))


class V41LM(nn.Module):
    def __init__(self, config: V41Config, ep_group=None, ep_buffers=None):
        super().__init__()
        c = self.config = config
        self.embed = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(V41Block(c, ep_group, ep_buffers) for _ in range(c.n_layer))
        self.head_mix = nn.Parameter(torch.zeros(c.hc_streams))
        self.norm = RMSNorm(c.hidden_size, c.rms_eps)
        self.lm_head = nn.Linear(c.hidden_size, c.vocab_size, bias=False)
        self.step = 0
        self.last_loss_metrics: dict = {}

    @torch.no_grad()
    def init_weights(self, std: float = 0.02):
        for n, p in self.named_parameters():
            if p.ndim >= 2:
                nn.init.normal_(p, std=std)
        self.head_mix.zero_()
        for m in self.modules():                     # gains, sinks and biases too: a meta-built model has no defaults
            if isinstance(m, HyperConnectionMix):
                nn.init.normal_(m.proj.weight, std=std)
                m.scale.fill_(0.01)
                m.base.zero_()
                m.base[2 * m.n:] = (torch.eye(m.n, device=m.base.device, dtype=m.base.dtype) * 4.0).flatten()   # near-identity mixing
            if isinstance(m, nn.LayerNorm):
                m.reset_parameters()
            if isinstance(m, RMSNorm):
                m.weight.fill_(0.0 if m.zero_centered else 1.0)
            if isinstance(m, SparseLatentAttention):
                m.sink.zero_()
            if isinstance(m, nn.Linear) and m.bias is not None:
                m.bias.zero_()

    def routers(self):
        return [b.ffn for b in self.layers]

    def forward(self, ids: torch.Tensor, labels: torch.Tensor | None = None):
        c = self.config
        B, S = ids.shape
        dt = torch.bfloat16 if ids.device.type == "cuda" else torch.float32
        x = self.embed(ids).to(dt)
        streams = x.unsqueeze(-2).expand(B, S, c.hc_streams, c.hidden_size).contiguous()
        cos, sin = rope_tables(S, c.rope_dim, c.rope_theta, ids.device)
        dense = self.step < c.dense_warmup_steps
        with torch.autocast(ids.device.type, dtype=dt, enabled=dt != torch.float32):
            for blk in self.layers:
                streams = blk(streams, cos, sin, dense)
            w = torch.softmax(self.head_mix.float(), 0)
            h = self.norm((streams.float() * w[:, None]).sum(-2).to(dt))
            logits = self.lm_head(h).float()
        if labels is None:
            return logits
        ce = F.cross_entropy(logits.flatten(0, 1), labels.flatten(), ignore_index=-1)
        kls = [b.attn.last_kl for b in self.layers if b.attn.last_kl is not None]
        kl = torch.stack(kls).mean() if kls else ce.new_zeros(())
        self.last_loss_metrics = {"cross entropy": ce.detach(), "indexer kl": kl.detach()}
        return ce + c.indexer_kl_weight * kl


from .protocol import attach_protocol  # noqa: E402  (after the classes it completes)

attach_protocol(V41LM)
