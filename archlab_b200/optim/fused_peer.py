"""ZeRO-1 Muon + AdamW whose collectives are fused into the optimizer kernels over NVLink peer
memory (``csrc/peer.cu``): the owner of a parameter slice loads that slice of every rank's
gradient buffer straight from peer memory, updates it in registers and stores the new bf16 weights
into every rank's shadow buffer - reduce-scatter, update and all-gather in ONE kernel per tensor,
with two device-side barriers per step for ordering.  Same update rules and ownership as
``optim.fused.FusedMuonAdamW`` / the reference's ``DistMuonAdamW``
(src/archlab/optimizers/speedrun.py:447-755), which remain the NCCL-decomposed baseline.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import native
from ..parallel import collectives as coll
from ..parallel.symm import PeerBarrier
from .fused import FusedMuonAdamW, polar_express_bf16
from .muon import adamw_update

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
native.register_signature("nga_peer_adamw", [_vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _f, _f, _f, _f, _f, _i, _i, _vp])
native.register_signature("nga_peer_muon_momentum", [_vp, _vp, _vp, _vp, _ll, _i, _ll, _i, _f, _vp])
native.register_signature("nga_peer_muon_apply", [_vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _f, _f, _vp])


class PeerMuonAdamW(FusedMuonAdamW):
    """Requires a ``ParamStore`` built with ``symmetric=True`` (gradients and shadows in symmetric
    memory).  Small / odd-shaped parameters (scalars, tiny gates) fall back to an NCCL all-reduce."""

    def __init__(self, model, store, **kw):
        super().__init__(model, store, **kw)
        if not getattr(store, "symmetric", False):
            raise ValueError("PeerMuonAdamW needs a symmetric ParamStore")
        self.barrier = PeerBarrier(model.lm_head.weight.device, self.pg)
        self.ws, self.rk = coll.world_size(self.pg), coll.rank(self.pg)

    # ------------------------------------------------------------------
    def _table_peer(self, p, g):
        name, _ = self._table_of[id(p)]
        sym_g, sym_s = self.store.sym_table_grad[name], self.store.sym_table_shadow[name]
        st = self.state.setdefault(id(p), {})
        rows = p.shape[0] // self.ws
        n = rows * p[0].numel()
        e0 = self.rk * n
        pslice = p.data[self.rk * rows:(self.rk + 1) * rows]
        if "exp_avg" not in st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(pslice)
            st["exp_avg_sq"] = torch.zeros_like(pslice)
        st["step"] += 1
        rc = native.lib().nga_peer_adamw(sym_g.ptr_array(), sym_s.ptr_array(), pslice.data_ptr(),
                                         st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(), e0, n, self.ws,
                                         g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"],
                                         st["step"], int(bool(g.get("cautious_weight_decay", False))),
                                         native.stream_ptr())
        native.check(rc, "nga_peer_adamw")

    def _adamw_group(self, g: dict) -> None:
        for p in g["params"]:
            is_table = id(p) in self._table_of and p.numel() % 4 == 0 and p.shape[0] % self.ws == 0 \
                and (p.numel() // self.ws) % 4 == 0
            if is_table:
                self._table_peer(p, g)
                continue
            st = self.state.setdefault(id(p), {})
            coll.all_reduce_avg(p.grad, self.pg)
            if "exp_avg" not in st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(p.data)
                st["exp_avg_sq"] = torch.zeros_like(p.data)
            st["step"] += 1
            adamw_update(p.data, p.grad, st["exp_avg"], st["exp_avg_sq"], step=st["step"], lr=g["lr"],
                         beta1=g["betas"][0], beta2=g["betas"][1], eps=g["eps"], wd=g["weight_decay"],
                         cautious=bool(g.get("cautious_weight_decay", False)))
            if id(p) in self._table_of:
                self._table_of[id(p)][1].copy_(p.data)

    def _muon_group(self, g: dict) -> None:
        shape, _ = self.store.locate(g["params"][0])
        sg = self.store.groups[shape]
        m, n = shape
        per = m * n
        L = native.lib()
        if per % 4 or n % 4 or min(m, n) < 64:
            # tiny matrices: replicated update after an NCCL all-reduce
            coll.all_reduce_avg(sg.grad, self.pg)
            st = self.state.setdefault(("muon", shape), {})
            from .fused import fused_muon_

            fused_muon_(sg.master, sg.grad, sg.shadow, st, momentum=g["momentum"],
                        lr=g["lr"] * max(1.0, m / n) ** 0.5, wd=g["weight_decay"],
                        beta2=g["beta2"] if g["beta2"] is not None else 0.0, ns_steps=g["ns_steps"])
            return
        sym_g, sym_s = self.store.sym_group_grad[shape], self.store.sym_group_shadow[shape]
        chunk = sg.master.size(0) // self.ws
        e0 = self.rk * chunk * per
        own = slice(self.rk * chunk, (self.rk + 1) * chunk)
        st = self.state.setdefault(("muon", shape), {})
        dev = sg.master.device
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros(chunk, m, n, dtype=torch.float32, device=dev)
            sshape = (chunk, m, 1) if m >= n else (chunk, 1, n)
            st["second_momentum_buffer"] = torch.zeros(sshape, dtype=torch.float32, device=dev)
            st["norm2"] = torch.zeros(chunk, dtype=torch.float32, device=dev)
            st["gn"] = torch.empty(chunk, m, n, dtype=torch.float32, device=dev)
        native.check(L.nga_peer_muon_momentum(sym_g.ptr_array(), st["gn"].data_ptr(),
                                              st["momentum_buffer"].data_ptr(), st["norm2"].data_ptr(), e0, chunk,
                                              per, self.ws, g["momentum"], native.stream_ptr()),
                     "nga_peer_muon_momentum")
        X = torch.empty(chunk, m, n, dtype=torch.bfloat16, device=dev)
        native.check(L.nga_muon_normalize(st["gn"].data_ptr(), st["norm2"].data_ptr(), X.data_ptr(), chunk, per,
                                          native.stream_ptr()), "nga_muon_normalize")
        X = polar_express_bf16(X, g["ns_steps"])
        per_row = m >= n
        red = n if per_row else m
        v_mean = torch.empty((chunk, m, 1) if per_row else (chunk, 1, n), dtype=torch.float32, device=dev)
        native.check(L.nga_sq_mean(X.data_ptr(), v_mean.data_ptr(), chunk, m, n, int(per_row), native.stream_ptr()),
                     "nga_sq_mean")
        beta2 = g["beta2"] if g["beta2"] is not None else 0.0
        v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * red).sqrt()
        sm = st["second_momentum_buffer"]
        sm.lerp_(v_mean, 1 - beta2)
        step_size = sm.clamp_min(1e-10).rsqrt()
        v_norm_new = ((v_mean * red) * step_size.square()).sum(dim=(-2, -1), keepdim=True).sqrt()
        scale = (step_size * (v_norm / v_norm_new.clamp_min(1e-10))).to(torch.bfloat16).float().contiguous()
        native.check(L.nga_peer_muon_apply(sg.master[own].data_ptr(), X.data_ptr(), scale.data_ptr(),
                                           sym_s.ptr_array(), e0, chunk, m, n, int(per_row), self.ws,
                                           g["lr"] * max(1.0, m / n) ** 0.5, g["weight_decay"],
                                           native.stream_ptr()), "nga_peer_muon_apply")

    @torch.no_grad()
    def step(self) -> None:
        self.barrier()          # every rank's backward has finished writing its gradient buffers
        for g in self.param_groups:
            if g["kind"] == "adamw":
                self._adamw_group(g)
            elif g["kind"] == "muon":
                self._muon_group(g)
            else:
                raise ValueError(f"unsupported optimizer kind {g['kind']!r}")
        self.barrier()          # every rank has read all gradients and written all shadows
        self._optimizer_step += 1
