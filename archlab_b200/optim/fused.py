"""Fused Muon + AdamW step over the engine's stacked parameter store (CUDA only).

Same update rules as ``optim.muon`` (which follows src/archlab/optimizers/speedrun.py:31-231), but:

* Muon groups are processed in place on the stacked ``(K, m, n)`` fp32 master / gradient buffers of
  ``ParamStore`` - no per-step ``torch.stack`` / copy-back;
* momentum, normalisation, variance statistics and the final update are one-pass CUDA kernels
  (``csrc/optim.cu``) that also write the bf16 shadow weights;
* the Newton-Schulz products run on the tcgen05 GEMM, batched over the K matrices;
* with a process group, gradients of a stacked group are reduce-scattered over K (each rank owns
  ``ceil(K / world)`` whole matrices: ZeRO-1 ownership as in ``DistMuonAdamW``) and the updated bf16
  shadows + fp32 masters are all-gathered; embedding-like tables are reduce-scattered by rows.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import native
from ..parallel import collectives as coll
from .muon import POLAR_EXPRESS_COEFFS, _mm, adamw_update

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
native.register_signature("nga_adamw", [_vp, _vp, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _i, _i, _vp])
native.register_signature("nga_muon_momentum", [_vp, _vp, _vp, _i, _ll, _f, _vp])
native.register_signature("nga_muon_normalize", [_vp, _vp, _vp, _i, _ll, _vp])
native.register_signature("nga_sq_mean", [_vp, _vp, _i, _i, _i, _i, _vp])
native.register_signature("nga_muon_apply", [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _vp])


def _s():
    return native.stream_ptr()


def fused_adamw_(p, g, m, v, shadow, *, step, lr, beta1, beta2, eps, wd, cautious=False):
    rc = native.lib().nga_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                shadow.data_ptr() if shadow is not None else None, p.numel(), lr, beta1,
                                beta2, eps, wd, step, int(cautious), _s())
    native.check(rc, "nga_adamw")


def polar_express_bf16(X: torch.Tensor, ns_steps: int) -> torch.Tensor:
    """X (K, m, n) bf16, already scaled to spectral norm <= 1; returns the orthogonalised stack."""
    tall = X.size(-2) > X.size(-1)
    for a, b, c in POLAR_EXPRESS_COEFFS[:ns_steps]:
        if tall:
            A = _mm(X, X, a_mn=True, b_mn=True)
            B = _mm(A, A, b_mn=False, aux=A, alpha=c, beta=b)
            X = _mm(X, B, b_mn=False, aux=X, alpha=1.0, beta=a)
        else:
            A = _mm(X, X, b_mn=False)
            B = _mm(A, A, b_mn=False, aux=A, alpha=c, beta=b)
            X = _mm(B, X, b_mn=True, aux=X, alpha=1.0, beta=a)
    return X


def fused_muon_(master, grad, shadow, state: dict, *, momentum, lr, wd, beta2, ns_steps):
    """In-place Muon step on stacked buffers ``(K, m, n)``; ``state`` holds the moment buffers."""
    K, m, n = master.shape
    per = m * n
    L = native.lib()
    if "momentum_buffer" not in state:
        state["momentum_buffer"] = torch.zeros_like(master)
        sshape = (K, m, 1) if m >= n else (K, 1, n)
        state["second_momentum_buffer"] = torch.zeros(sshape, dtype=torch.float32, device=master.device)
        state["norm2"] = torch.zeros(K, dtype=torch.float32, device=master.device)
    if per % 4 or n % 4 or min(m, n) < 64:
        # tiny matrices (e.g. the 10 x 12 value-embedding gates): plain PyTorch path
        from .muon import muon_update

        muon_update(grad, master, state["momentum_buffer"], state["second_momentum_buffer"], momentum=momentum,
                    lr=lr, wd=wd, beta2=beta2, ns_steps=ns_steps, red_dim=-1 if m >= n else -2, bf16=True)
        shadow.copy_(master)
        return
    native.check(L.nga_muon_momentum(grad.data_ptr(), state["momentum_buffer"].data_ptr(),
                                     state["norm2"].data_ptr(), K, per, momentum, _s()), "nga_muon_momentum")
    X = torch.empty(K, m, n, dtype=torch.bfloat16, device=master.device)
    native.check(L.nga_muon_normalize(grad.data_ptr(), state["norm2"].data_ptr(), X.data_ptr(), K, per, _s()),
                 "nga_muon_normalize")
    X = polar_express_bf16(X, ns_steps)
    per_row = m >= n
    red = n if per_row else m
    v_mean = torch.empty((K, m, 1) if per_row else (K, 1, n), dtype=torch.float32, device=master.device)
    native.check(L.nga_sq_mean(X.data_ptr(), v_mean.data_ptr(), K, m, n, int(per_row), _s()), "nga_sq_mean")
    # NorMuon statistics on the small (K, m) / (K, n) vectors
    v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * red).sqrt()
    sm = state["second_momentum_buffer"]
    sm.lerp_(v_mean, 1 - beta2)
    step_size = sm.clamp_min(1e-10).rsqrt()
    v_norm_new = ((v_mean * red) * step_size.square()).sum(dim=(-2, -1), keepdim=True).sqrt()
    scale = (step_size * (v_norm / v_norm_new.clamp_min(1e-10))).contiguous()
    # the reference applies the scale in bf16
    scale = scale.to(torch.bfloat16).float()
    native.check(L.nga_muon_apply(master.data_ptr(), X.data_ptr(), scale.data_ptr(), shadow.data_ptr(), K, m, n,
                                  int(per_row), lr, wd, _s()), "nga_muon_apply")


class FusedMuonAdamW:
    """Optimizer over a ``ParamStore`` (single GPU, or ZeRO-1 over ``group``)."""

    def __init__(self, model, store, *, unembedding_lr=0.004, embedding_lr=0.2, matrix_lr=0.02,
                 weight_decay=0.0, scalar_lr=0.5, group=None):
        from .setup import base_parameter_groups

        self.model, self.store, self.pg = model, store, group
        self.param_groups = base_parameter_groups(model, unembedding_lr=unembedding_lr, embedding_lr=embedding_lr,
                                                  matrix_lr=matrix_lr, weight_decay=weight_decay,
                                                  scalar_lr=scalar_lr)
        for g in self.param_groups:
            g["initial_lr"] = g["lr"]
        self.state: dict = {}
        self._table_of = {id(p): (name, sh) for name, (p, sh) in store.tables.items()}
        self._optimizer_step = 0

    # ------------------------------------------------------------------
    def _adamw_group(self, g: dict) -> None:
        ws, rk = coll.world_size(self.pg), coll.rank(self.pg)
        for p in g["params"]:
            st = self.state.setdefault(id(p), {})
            is_table = id(p) in self._table_of and p.numel() % 4 == 0
            sharded = ws > 1 and is_table and p.shape[0] % ws == 0
            if sharded:
                rows = p.shape[0] // ws
                pslice = p.data[rk * rows:(rk + 1) * rows]
                gslice = st["grad_slice"]
                st["rs_handle"].wait()
                shadow = self._table_of[id(p)][1]
                sslice = shadow[rk * rows:(rk + 1) * rows]
            else:
                pslice, gslice = p.data, p.grad
                sslice = self._table_of[id(p)][1] if is_table else None
                if ws > 1:
                    st["rs_handle"].wait()
            if "exp_avg" not in st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(pslice)
                st["exp_avg_sq"] = torch.zeros_like(pslice)
            st["step"] += 1
            kw = dict(step=st["step"], lr=g["lr"], beta1=g["betas"][0], beta2=g["betas"][1], eps=g["eps"],
                      wd=g["weight_decay"], cautious=bool(g.get("cautious_weight_decay", False)))
            if is_table:
                fused_adamw_(pslice, gslice, st["exp_avg"], st["exp_avg_sq"], sslice, **kw)
            else:
                adamw_update(pslice, gslice, st["exp_avg"], st["exp_avg_sq"], **kw)
            if sharded:
                self._gathers.append(coll.all_gather_into(shadow, sslice, self.pg, async_op=True))

    def _muon_group(self, g: dict) -> None:
        p0 = g["params"][0]
        shape, _ = self.store.locate(p0)
        sg = self.store.groups[shape]
        if len(sg.params) != len(g["params"]):
            raise RuntimeError("Muon group does not cover its stacked buffer")
        st = self.state.setdefault(("muon", shape), {})
        m, n = shape
        ws, rk = coll.world_size(self.pg), coll.rank(self.pg)
        kw = dict(momentum=g["momentum"], lr=g["lr"] * max(1.0, m / n) ** 0.5, wd=g["weight_decay"],
                  beta2=g["beta2"] if g["beta2"] is not None else 0.0, ns_steps=g["ns_steps"])
        if ws == 1:
            fused_muon_(sg.master, sg.grad, sg.shadow, st, **kw)
            return
        chunk = sg.master.size(0) // ws
        st["rs_handle"].wait()
        own = slice(rk * chunk, (rk + 1) * chunk)
        fused_muon_(sg.master[own], st["grad_chunk"], sg.shadow[own], st, **kw)
        self._gathers.append(coll.all_gather_into(sg.shadow, sg.shadow[own], self.pg, async_op=True))

    @torch.no_grad()
    def step(self) -> None:
        """Phase 1 launches every gradient reduction, phase 2 updates group by group as its reduction
        lands (later reductions overlap earlier updates) and launches the shadow all-gathers, phase 3
        waits for the gathers: the three-phase shape of the reference's distributed optimizer
        (src/archlab/optimizers/speedrun.py:729-755)."""
        self._gathers = []
        if coll.world_size(self.pg) > 1:
            self._launch_reductions()
        for g in self.param_groups:
            if g["kind"] == "adamw":
                self._adamw_group(g)
            elif g["kind"] == "muon":
                self._muon_group(g)
            else:
                raise ValueError(f"unsupported optimizer kind {g['kind']!r}")
        for h in self._gathers:
            h.wait()
        self._optimizer_step += 1

    # ------------------------------------------------------------------
    def _launch_reductions(self) -> None:
        ws = coll.world_size(self.pg)
        for g in self.param_groups:
            if g["kind"] == "muon":
                shape, _ = self.store.locate(g["params"][0])
                sg = self.store.groups[shape]
                st = self.state.setdefault(("muon", shape), {})
                chunk = sg.master.size(0) // ws
                if "grad_chunk" not in st:
                    st["grad_chunk"] = torch.empty(chunk, *shape, dtype=torch.float32, device=sg.grad.device)
                st["rs_handle"] = coll.reduce_scatter_avg(st["grad_chunk"], sg.grad, self.pg, async_op=True)
            else:
                for p in g["params"]:
                    st = self.state.setdefault(id(p), {})
                    is_table = id(p) in self._table_of and p.numel() % 4 == 0
                    if is_table and p.shape[0] % ws == 0:
                        rows = p.shape[0] // ws
                        if "grad_slice" not in st:
                            st["grad_slice"] = torch.empty(rows, *p.shape[1:], dtype=torch.float32,
                                                           device=p.device)
                        st["rs_handle"] = coll.reduce_scatter_avg(st["grad_slice"], p.grad, self.pg, async_op=True)
                    else:
                        st["rs_handle"] = coll.all_reduce_avg(p.grad, self.pg, async_op=True)

    def gather_master(self) -> None:
        """All-gather the fp32 master weights (needed before a full checkpoint; between steps only the
        owner's slice of each master buffer is current)."""
        ws, rk = coll.world_size(self.pg), coll.rank(self.pg)
        if ws == 1:
            return
        for sg in self.store.groups.values():
            chunk = sg.master.size(0) // ws
            coll.all_gather_into(sg.master, sg.master[rk * chunk:(rk + 1) * chunk].clone(), self.pg)
        for p, _ in self.store.tables.values():
            if p.numel() % 4 == 0 and p.shape[0] % ws == 0:
                rows = p.shape[0] // ws
                coll.all_gather_into(p.data, p.data[rk * rows:(rk + 1) * rows].clone(), self.pg)

    def state_dict(self) -> dict:
        return {"state": self.state, "step": self._optimizer_step,
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}
