"""Fused sm_100a execution engine for the speedrun GPT.

``FusedGPTEngine`` drives the parameters of a ``models.nanochat.GPT`` through hand-written kernels:
tcgen05 GEMMs with fused epilogues (residual add, ReLU^2, ReLU^2 backward, fp32 gradient
accumulation), tcgen05 attention forward / key-owned backward, and one-pass memory-bound kernels
for embedding+norm+smear, lambda-mix+norm, QKV post-processing (RoPE, QK-norm, value-embedding gate)
and the chunked lm_head + soft-capped cross entropy (forward and backward in the same pass, so the
``tokens x vocab`` logits never exist at full size).  The backward pass is written by hand; PyTorch
autograd is not involved on this path.

Memory layout: all same-shape trunk matrices live in ONE stacked fp32 master buffer ``(K, m, n)``
with a matching fp32 gradient buffer and a bf16 shadow used by the GEMMs (q, k, v, proj of a layer
are adjacent, so the fused QKV weight is a contiguous ``[3C, C]`` slice of the shadow).  The
``nn.Parameter`` objects of the module are re-pointed at views of these buffers, so optimizers,
checkpoints and the eager model see the same storage.  The stacked layout is exactly what the
Muon step consumes (src/archlab/optimizers/speedrun.py:406-434 stacks per step instead).

The reference runs this model through ``torch.compile`` + FlashAttention-4 + cuBLAS
(src/archlab/speedrun/base_train.py:1240, 1812-1836).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..ops import native, trunk
from ..ops.gemm import EPI_ATOMIC_ADD, EPI_AXPBY, EPI_MUL_DRELU2, EPI_RELU2, EPI_SCALE, gemm
from .nanochat import GPT, GPTConfig, has_ve


@dataclass
class StackedGroup:
    """Same-shape matrices stacked along dim 0."""
    shape: tuple[int, int]
    master: torch.Tensor     # (K, m, n) fp32
    grad: torch.Tensor       # (K, m, n) fp32
    shadow: torch.Tensor     # (K, m, n) bf16
    params: list             # the nn.Parameters, in stacking order


class ParamStore:
    """Re-homes the module's parameters into stacked / flat buffers (see module docstring)."""

    def __init__(self, model: GPT, world: int = 1, symmetric: bool = False, group=None):
        """``symmetric`` places gradient and shadow buffers in NVLink symmetric memory (same offset on
        every rank, peer-mapped) for the fused collective kernels.  ``world`` pads every stacked group to a multiple of the data-parallel world size so that
        whole matrices can be reduce-scattered / all-gathered without staging copies."""
        cfg = model.config
        dev = model.lm_head.weight.device
        self.world = world
        self.symmetric = symmetric
        self.sym_group_grad, self.sym_group_shadow = {}, {}
        self.sym_table_grad, self.sym_table_shadow = {}, {}
        if symmetric:
            from ..parallel.symm import symm_zeros

        def alloc(shape, dtype, registry, key):
            if not symmetric:
                return torch.zeros(shape, dtype=dtype, device=dev)
            st = symm_zeros(tuple(shape), dtype, dev, group)
            registry[key] = st
            return st.tensor

        self.groups: dict[tuple[int, int], StackedGroup] = {}
        order: dict[tuple[int, int], list] = {}
        for block in model.transformer.h:
            attn, mlp = block.attn, block.mlp
            mats = [attn.c_q.weight, attn.c_k.weight, attn.c_v.weight, attn.c_proj.weight,
                    mlp.c_fc.weight, mlp.c_proj.weight]
            if hasattr(attn, "c_k2"):                      # 2-simplicial layer: second key / value branch
                mats += [attn.c_k2.weight, attn.c_v2.weight]
            if attn.ve_gate is not None:
                mats.append(attn.ve_gate.weight)
            for p in mats:
                order.setdefault(tuple(p.shape), []).append(p)
        for shape, plist in order.items():
            K = (len(plist) + world - 1) // world * world
            master = torch.zeros(K, *shape, dtype=torch.float32, device=dev)
            for i, p in enumerate(plist):
                master[i].copy_(p.data)
                p.data = master[i]
            grad = alloc(master.shape, torch.float32, self.sym_group_grad, shape)
            for i, p in enumerate(plist):
                p.grad = grad[i]
            shadow = alloc(master.shape, torch.bfloat16, self.sym_group_shadow, shape)
            shadow.copy_(master)
            self.groups[shape] = StackedGroup(shape, master, grad, shadow, plist)
        # embedding-like tables: fp32 master + fp32 grad + bf16 shadow each
        self.tables: dict[str, tuple[torch.nn.Parameter, torch.Tensor]] = {}
        names = [("wte", model.transformer.wte.weight), ("lm_head", model.lm_head.weight)]
        names += [(f"ve{i}", ve.weight) for i, ve in model.value_embeds.items()]
        for name, p in names:
            p.grad = alloc(p.data.shape, torch.float32, self.sym_table_grad, name)
            sh = alloc(p.data.shape, torch.bfloat16, self.sym_table_shadow, name)
            sh.copy_(p.data)
            self.tables[name] = (p, sh)
        # scalars stay fp32 and are read by the kernels directly
        self.scalars = [model.resid_lambdas, model.x0_lambdas, model.smear_gate.weight, model.smear_lambda,
                        model.backout_lambda]
        for p in self.scalars:
            p.grad = torch.zeros_like(p.data)
        self._index = {id(p): (shape, i) for shape, g in self.groups.items() for i, p in enumerate(g.params)}

    def locate(self, p) -> tuple[tuple[int, int], int]:
        return self._index[id(p)]

    def shadow_of(self, p) -> torch.Tensor:
        shape, i = self.locate(p)
        return self.groups[shape].shadow[i]

    def grad_of(self, p) -> torch.Tensor:
        shape, i = self.locate(p)
        return self.groups[shape].grad[i]

    def table_shadow(self, name: str) -> torch.Tensor:
        return self.tables[name][1]

    @torch.no_grad()
    def refresh_shadows(self) -> None:
        """bf16 copies of every master weight (called after each optimizer step)."""
        for g in self.groups.values():
            if g.master.numel() % 4 == 0:
                trunk.cast_to_bf16_(g.shadow, g.master)
            else:
                g.shadow.copy_(g.master)
        for p, sh in self.tables.values():
            trunk.cast_to_bf16_(sh, p.data)

    @torch.no_grad()
    def zero_grads(self) -> None:
        for g in self.groups.values():
            g.grad.zero_()
        for p, _ in self.tables.values():
            p.grad.zero_()
        for p in self.scalars:
            p.grad.zero_()


class FusedGPTEngine:
    """Forward + hand-written backward of the speedrun GPT on one B200.

    ``forward_backward(idx, targets, gscale)`` accumulates ``gscale * d(sum of token losses)`` into the
    fp32 gradient buffers and returns the summed loss of the micro-batch (a 0-d device tensor, not
    scaled).  Call ``store.zero_grads()`` at the start of a step and ``store.refresh_shadows()`` after
    the optimizer has changed the master weights.
    """

    def __init__(self, model: GPT, *, head_chunk: int = 8192, world: int = 1, symmetric: bool = False,
                 group=None):
        cfg = model.config
        if cfg.head_dim != 128:
            raise ValueError("the fused engine supports head_dim 128")
        if cfg.n_embd % 8 or cfg.padded_vocab != cfg.vocab_size:
            raise ValueError("n_embd must be a multiple of 8 and the vocabulary a multiple of 64")
        if model.lm_head.weight.device.type != "cuda":
            raise ValueError("the fused engine needs CUDA parameters")
        native.lib()   # fail loudly if the native library is missing
        self.model, self.cfg = model, cfg
        self.store = ParamStore(model, world, symmetric, group)
        # A 2-simplicial layer keeps its module as the statement of the mixer (five projections, RoPE + norms, the
        # simplicial kernels) and runs under autograd inside the otherwise hand-written step: its linears go onto the
        # tcgen05 GEMMs, its weight gradients accumulate into the store's fp32 buffers through ``p.grad``.
        self.simplicial = set(cfg.simplicial_layers)
        if self.simplicial:
            from ..ops.native_linear import convert_linears

            for i in self.simplicial:
                convert_linears(model.transformer.h[i].attn, min_features=64)
        self.head_chunk = head_chunk
        dev = model.lm_head.weight.device
        self.dev = dev
        T = cfg.sequence_len
        cos, sin = model.cos[:T].float().to(dev).contiguous(), model.sin[:T].float().to(dev).contiguous()
        # tables hold the bf16-rounded values the eager model multiplies with
        if cfg.compute_dtype == torch.bfloat16:
            self.cosT, self.sinT = cos, sin
        else:
            self.cosT, self.sinT = cos.bfloat16().float(), sin.bfloat16().float()
        self._ws: dict = {}
        H, Hkv, C = cfg.n_head, cfg.n_kv_head, cfg.n_embd
        self.qkv_contig = Hkv == H
        if not self.qkv_contig:
            L, QC = cfg.n_layer, (H + 2 * Hkv) * cfg.head_dim
            self.wqkv_shadow = torch.empty(L, QC, C, dtype=torch.bfloat16, device=dev)
            self.wqkv_grad = torch.zeros(L, QC, C, dtype=torch.float32, device=dev)
            self._fill_wqkv()

    # ------------------------------------------------------------------ weights
    def _fill_wqkv(self) -> None:
        if self.qkv_contig:
            return
        for i, block in enumerate(self.model.transformer.h):
            a = block.attn
            torch.cat([self.store.shadow_of(a.c_q.weight), self.store.shadow_of(a.c_k.weight),
                       self.store.shadow_of(a.c_v.weight)], dim=0, out=self.wqkv_shadow[i])

    def refresh_shadows(self) -> None:
        self.store.refresh_shadows()
        self._fill_wqkv()

    def _wqkv(self, i: int):
        """(bf16 fused QKV weight [QC, C], fp32 gradient view [QC, C]) of layer i."""
        if not self.qkv_contig:
            return self.wqkv_shadow[i], self.wqkv_grad[i]
        a = self.model.transformer.h[i].attn
        shape, k = self.store.locate(a.c_q.weight)
        g = self.store.groups[shape]
        C = self.cfg.n_embd
        return g.shadow[k:k + 3].view(3 * C, C), g.grad[k:k + 3].view(3 * C, C)

    def _scatter_wqkv_grads(self) -> None:
        if self.qkv_contig:
            return
        cfg = self.cfg
        nq, nk = cfg.n_head * cfg.head_dim, cfg.n_kv_head * cfg.head_dim
        for i, block in enumerate(self.model.transformer.h):
            a = block.attn
            g = self.wqkv_grad[i]
            self.store.grad_of(a.c_q.weight).add_(g[:nq])
            self.store.grad_of(a.c_k.weight).add_(g[nq:nq + nk])
            self.store.grad_of(a.c_v.weight).add_(g[nq + nk:])
        self.wqkv_grad.zero_()

    # ------------------------------------------------------------------ forward
    def _forward(self, idx: torch.Tensor) -> dict:
        """Runs the trunk; returns the saved activations needed by the backward."""
        cfg, st, m = self.cfg, self.store, self.model
        B, T = idx.shape
        C, L = cfg.n_embd, cfg.n_layer
        H, Hkv, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        idx_flat = idx.reshape(-1)
        sv: dict = {"idx": idx_flat, "B": B, "T": T}
        x0, sv["smear_pre"] = trunk.embed_fwd(idx_flat, st.table_shadow("wte"), m.smear_gate.weight.data.view(-1),
                                              m.smear_lambda.data, T)
        xs, x1s, n1s, qkvs, ys, lses, x2s, n2s, acts, rstds, gps = ([] for _ in range(11))
        xs.append(x0)
        x = x0
        for i, block in enumerate(m.transformer.h):
            x1, n1 = trunk.mix_norm_fwd(x, x0, m.resid_lambdas.data[i:i + 1], m.x0_lambdas.data[i:i + 1])
            if i in self.simplicial:
                leaf = n1.detach().requires_grad_(True)
                with torch.enable_grad():
                    mixed = block.attn(leaf.view(B, T, C), None, m.cos[:T].to(n1.dtype), m.sin[:T].to(n1.dtype), m.window_sizes[i])
                x2 = x1 + mixed.detach().reshape(-1, C)
                sv.setdefault("simplicial", {})[i] = (leaf, mixed)
                _, n2 = trunk.mix_norm_fwd(x2)
                act = gemm(n2, st.shadow_of(block.mlp.c_fc.weight), epi=EPI_RELU2)
                x3 = gemm(act, st.shadow_of(block.mlp.c_proj.weight), aux=x2, epi=EPI_AXPBY, alpha=1.0, beta=1.0)
                for lst, v in ((xs, x3), (x1s, x1), (n1s, n1), (qkvs, None), (ys, None), (lses, None), (x2s, x2),
                               (n2s, n2), (acts, act), (rstds, None), (gps, None)):
                    lst.append(v)
                x = x3
                continue
            wqkv, _ = self._wqkv(i)
            qkv = gemm(n1, wqkv)
            ve_name = f"ve{i}"
            has = ve_name in st.tables
            rstd, gate_pre = trunk.qkv_post_fwd(
                qkv, self.cosT, self.sinT, 1.2, idx_flat, st.table_shadow(ve_name) if has else None,
                block.attn.ve_gate.weight.data if has else None, n1, T, H, Hkv, D)
            window = m.window_sizes[i]
            y, lse = trunk.attn_fwd(qkv, B, T, H, Hkv, D, -1 if window >= T else window)
            x2 = gemm(y, st.shadow_of(block.attn.c_proj.weight), aux=x1, epi=EPI_AXPBY, alpha=1.0, beta=1.0)
            _, n2 = trunk.mix_norm_fwd(x2)
            act = gemm(n2, st.shadow_of(block.mlp.c_fc.weight), epi=EPI_RELU2)
            x3 = gemm(act, st.shadow_of(block.mlp.c_proj.weight), aux=x2, epi=EPI_AXPBY, alpha=1.0, beta=1.0)
            for lst, v in ((xs, x3), (x1s, x1), (n1s, n1), (qkvs, qkv), (ys, y), (lses, lse), (x2s, x2),
                           (n2s, n2), (acts, act), (rstds, rstd), (gps, gate_pre)):
                lst.append(v)
            x = x3
        xb = xs[L // 2 + 1]
        xf, nf = trunk.mix_norm_fwd(x, xb, None, m.backout_lambda.data, 1.0, -1.0)
        sv.update(xs=xs, x1=x1s, n1=n1s, qkv=qkvs, y=ys, lse=lses, x2=x2s, n2=n2s, act=acts, rstd=rstds,
                  gate_pre=gps, xf=xf, nf=nf)
        return sv

    @torch.no_grad()
    def logits(self, idx: torch.Tensor) -> torch.Tensor:
        """Soft-capped logits [B, T, V] in fp32 (evaluation / tests; materialises the full tensor)."""
        sv = self._forward(idx)
        raw = gemm(sv["nf"], self.store.table_shadow("lm_head")).float()
        cap = self.cfg.logit_softcap
        return (cap * torch.tanh(raw / cap)).view(idx.size(0), idx.size(1), -1)

    # ------------------------------------------------------------------ head (forward + backward)
    def _head(self, sv: dict, targets: torch.Tensor, gscale: float) -> tuple[torch.Tensor, torch.Tensor]:
        cfg, st = self.cfg, self.store
        nf = sv["nf"]
        Nt = nf.size(0)
        wlm = st.table_shadow("lm_head")
        glm = st.tables["lm_head"][0].grad
        tflat = targets.reshape(-1)
        dnf = torch.empty_like(nf)
        losses = torch.empty(Nt, dtype=torch.float32, device=nf.device)
        ch = self.head_chunk
        for s in range(0, Nt, ch):
            e = min(Nt, s + ch)
            logits = gemm(nf[s:e], wlm)
            losses[s:e] = trunk.softcap_ce_(logits, tflat[s:e], gscale, cfg.logit_softcap)
            gemm(logits, wlm, b_mn=True, out=dnf[s:e])
            gemm(logits, nf[s:e], a_mn=True, b_mn=True, out=glm, epi=EPI_ATOMIC_ADD)
        return losses.sum(), dnf

    # ------------------------------------------------------------------ backward
    def _backward(self, sv: dict, dnf: torch.Tensor) -> None:
        cfg, st, m = self.cfg, self.store, self.model
        B, T, idx_flat = sv["B"], sv["T"], sv["idx"]
        L = cfg.n_layer
        H, Hkv, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        xs, x0 = sv["xs"], sv["xs"][0]
        xb = xs[L // 2 + 1]
        Nt, C = x0.shape
        dxb = torch.empty_like(x0)
        dx0 = torch.empty_like(x0)
        # final: xf = x_L - lambda * xb ; nf = rmsnorm(xf)
        dx = trunk.norm_bwd_mix(sv["xf"], dnf, None, None, m.backout_lambda.data, xs[L], xb, dxb, True,
                                None, m.backout_lambda.grad, 1.0, -1.0)
        dq_acc = torch.empty(Nt, H * D, dtype=torch.float32, device=x0.device)
        delta = torch.empty(B, H, T, dtype=torch.float32, device=x0.device)
        for i in range(L - 1, -1, -1):
            block = m.transformer.h[i]
            if i == L // 2:
                trunk.axpby_(dx, dxb)          # gradient of the backout read of this block's output
            w_p2, g_p2 = st.shadow_of(block.mlp.c_proj.weight), st.grad_of(block.mlp.c_proj.weight)
            w_fc, g_fc = st.shadow_of(block.mlp.c_fc.weight), st.grad_of(block.mlp.c_fc.weight)
            w_o, g_o = st.shadow_of(block.attn.c_proj.weight), st.grad_of(block.attn.c_proj.weight)
            act, n2, x2, y = sv["act"][i], sv["n2"][i], sv["x2"][i], sv["y"][i]
            # ---- MLP
            dh = gemm(dx, w_p2, b_mn=True, aux=act, epi=EPI_MUL_DRELU2)
            gemm(dx, act, a_mn=True, b_mn=True, out=g_p2, epi=EPI_ATOMIC_ADD)
            dn2 = gemm(dh, w_fc, b_mn=True)
            gemm(dh, n2, a_mn=True, b_mn=True, out=g_fc, epi=EPI_ATOMIC_ADD)
            del dh
            dx2 = trunk.norm_bwd(x2, dn2, dx)
            if i in self.simplicial:
                leaf, mixed = sv["simplicial"].pop(i)
                with torch.enable_grad():
                    mixed.backward(dx2.view_as(mixed))        # weight gradients land in the store through p.grad
                dn1 = leaf.grad
                dx = trunk.norm_bwd_mix(sv["x1"][i], dn1, dx2, m.resid_lambdas.data[i:i + 1],
                                        m.x0_lambdas.data[i:i + 1], xs[i], x0, dx0, i == L - 1,
                                        m.resid_lambdas.grad[i:i + 1], m.x0_lambdas.grad[i:i + 1])
                for k in ("act", "n2", "x2", "n1", "x1"):
                    sv[k][i] = None
                continue
            # ---- attention
            dy = gemm(dx2, w_o, b_mn=True)
            gemm(dx2, y, a_mn=True, b_mn=True, out=g_o, epi=EPI_ATOMIC_ADD)
            window = m.window_sizes[i]
            qkv = sv["qkv"][i]
            dqkv = trunk.attn_bwd(qkv, y, dy, sv["lse"][i], B, T, H, Hkv, D, -1 if window >= T else window,
                                  dq_acc, delta)
            ve_name = f"ve{i}"
            has = ve_name in st.tables
            dgp = trunk.qkv_post_bwd(dqkv, qkv, self.cosT, self.sinT, 1.2, idx_flat,
                                     st.table_shadow(ve_name) if has else None, sv["rstd"][i],
                                     sv["gate_pre"][i], st.tables[ve_name][0].grad if has else None,
                                     T, H, Hkv, D)
            wqkv, gqkv = self._wqkv(i)
            n1 = sv["n1"][i]
            dn1 = gemm(dqkv, wqkv, b_mn=True)
            gemm(dqkv, n1, a_mn=True, b_mn=True, out=gqkv, epi=EPI_ATOMIC_ADD)
            if has:
                trunk.gate_bwd(dn1, n1, dgp, block.attn.ve_gate.weight.data, st.grad_of(block.attn.ve_gate.weight))
            dx = trunk.norm_bwd_mix(sv["x1"][i], dn1, dx2, m.resid_lambdas.data[i:i + 1],
                                    m.x0_lambdas.data[i:i + 1], xs[i], x0, dx0, i == L - 1,
                                    m.resid_lambdas.grad[i:i + 1], m.x0_lambdas.grad[i:i + 1])
            # free this layer's activations early
            for k in ("act", "n2", "x2", "y", "qkv", "n1", "x1", "lse", "rstd", "gate_pre"):
                sv[k][i] = None
        trunk.axpby_(dx, dx0)                  # x0 feeds layer 0 both as x and as x0
        wte_p = st.tables["wte"][0]
        trunk.embed_bwd(idx_flat, st.table_shadow("wte"), m.smear_gate.weight.data.view(-1), m.smear_lambda.data,
                        sv["smear_pre"], dx, wte_p.grad, m.smear_gate.weight.grad.view(-1), m.smear_lambda.grad, T)

    def forward_backward(self, idx: torch.Tensor, targets: torch.Tensor, gscale: float) -> torch.Tensor:
        with torch.no_grad():
            sv = self._forward(idx)
            loss_sum, dnf = self._head(sv, targets, gscale)
            self._backward(sv, dnf)
        return loss_sum

    def finish_step(self) -> None:
        """Fold auxiliary gradient buffers into the parameters' ``.grad`` (GQA layouts only)."""
        self._scatter_wqkv_grads()
