"""Optimizer-state sharding (ZeRO-1/2) over a data-parallel group on flat buffers.

Parameters and gradients of the model become views into two flat buffers in the compute dtype.  One
step: reduce-scatter of the flat gradient (every rank receives the sum of its 1/DP slice), fused AdamW
on the rank's fp32 master slice (one kernel per slice on sm_100a; it also writes the compute-dtype
copy), all-gather of the updated parameter slices.  With 180 GB per GPU the compute-dtype parameters
stay resident - only the fp32 master and the two moments (12 bytes per parameter) are divided by DP,
which is the part of the reference's FSDP/distributed-optimizer arrangement that saves memory
(src/archlab/megatron/qwen38_flash_next_config.py:216-221 enables the distributed optimizer with
overlapped parameter gather).

Gradients: with fp32 parameters (CPU tests) ``p.grad`` is a view of the flat gradient buffer.  With
bf16 / fp16 parameters the flat gradient buffer is fp32 ("main grads"): a post-accumulate hook adds every
micro-batch's low-precision ``p.grad`` into the fp32 view and drops it, so micro-batch accumulation, the
tensor- / context-parallel all-reduces over replicated ranges and the data-parallel reduce-scatter all
sum in fp32, and the gradient norm is taken from that sum (Megatron's bf16 path does the same).

Parameters with two or more dimensions are decayed; they are laid out first so that a slice meets at
most one boundary between decayed and undecayed ranges.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel import collectives as coll


class ZeroAdamW:
    def __init__(self, params, *, lr: float, weight_decay: float = 0.0, betas=(0.9, 0.95), eps: float = 1e-8,
                 group=None, align: int = 128, main_grads_fp32: bool | None = None):
        params = [p for p in params if p.requires_grad]
        self.group = group
        self.world, self.rank = coll.world_size(group), coll.rank(group)
        if group is None and self.world > 1 and not getattr(self, "_allow_world", True):
            raise ValueError("pass the data-parallel group")
        decayed = [p for p in params if p.dim() >= 2]
        plain = [p for p in params if p.dim() < 2]
        self.params = decayed + plain
        dev, dt = self.params[0].device, self.params[0].dtype
        pad = lambda n, a: (n + a - 1) // a * a
        n_dec = pad(sum(p.numel() for p in decayed), 4)
        n_all = pad(n_dec + sum(p.numel() for p in plain), align * self.world)
        self.n_decayed, self.numel = n_dec, n_all
        self.flat_p = torch.zeros(n_all, dtype=dt, device=dev)
        if main_grads_fp32 is None:
            main_grads_fp32 = dt in (torch.bfloat16, torch.float16)
        self.main_grads = bool(main_grads_fp32) and dt != torch.float32
        gdt = torch.float32 if self.main_grads else dt
        self.flat_g = torch.zeros(n_all, dtype=gdt, device=dev)
        off = 0
        for i, p in enumerate(self.params):
            if i == len(decayed):
                off = n_dec
            n = p.numel()
            self.flat_p[off:off + n].copy_(p.detach().reshape(-1))
            p.data = self.flat_p[off:off + n].view_as(p)
            if self.main_grads:
                p.grad = None
                p.register_post_accumulate_grad_hook(self._fold_into_main_grad(self.flat_g[off:off + n].view_as(p)))
            else:
                p.grad = self.flat_g[off:off + n].view_as(p)
            off += n
        self.shard = n_all // self.world
        lo = self.rank * self.shard
        self.lo, self.hi = lo, lo + self.shard
        self.master = self.flat_p[lo:self.hi].float()
        self.m, self.v = torch.zeros_like(self.master), torch.zeros_like(self.master)
        self.g32 = torch.empty_like(self.master)
        self.g_shard = torch.empty(self.shard, dtype=gdt, device=dev)
        self.lr, self.wd, self.betas, self.eps, self.t = lr, weight_decay, betas, eps, 0

    # -- gradient pieces ---------------------------------------------------------------------------
    @staticmethod
    def _fold_into_main_grad(main):
        def hook(param):
            main.add_(param.grad)
            param.grad = None
        return hook

    def zero_grad(self) -> None:
        self.flat_g.zero_()
        if self.main_grads:
            for p in self.params:
                p.grad = None
            return
        for p in self.params:                                    # autograd may have replaced the views
            if p.grad is None or p.grad.data_ptr() != self._grad_ptr(p):
                p.grad = self._grad_view(p)

    def _offsets(self):
        if not hasattr(self, "_off"):
            self._off, off, seen_plain = {}, 0, False
            for p in self.params:
                if p.dim() < 2 and not seen_plain:
                    off, seen_plain = self.n_decayed, True
                self._off[p] = off
                off += p.numel()
        return self._off

    def _grad_view(self, p):
        o = self._offsets()[p]
        return self.flat_g[o:o + p.numel()].view_as(p)

    def _grad_ptr(self, p):
        return self.flat_g.data_ptr() + self._offsets()[p] * self.flat_g.element_size()

    def range_of(self, params) -> tuple[int, int]:
        """Smallest flat range covering ``params`` (for one all-reduce over a replicated sub-range)."""
        offs = self._offsets()
        return min(offs[p] for p in params), max(offs[p] + p.numel() for p in params)

    def reduce_gradients(self) -> None:
        """Sum of the flat gradient over the group; this rank keeps its slice in fp32."""
        if self.world == 1:
            self.g32.copy_(self.flat_g[self.lo:self.hi])
            return
        if dist.get_backend(self.group) == "nccl":
            dist.reduce_scatter_tensor(self.g_shard, self.flat_g, group=self.group)
        else:
            tmp = self.flat_g.clone()
            dist.all_reduce(tmp, group=self.group)
            self.g_shard.copy_(tmp[self.lo:self.hi])
        self.g32.copy_(self.g_shard)

    def grad_sq_norm(self, ranges=None) -> torch.Tensor:
        """Sum of squares of this rank's reduced slice, optionally only inside the given flat ranges
        (add over the group for the global figure)."""
        if ranges is None:
            return self.g32.pow(2).sum()
        total = torch.zeros((), device=self.g32.device)
        for a, b in ranges:
            a, b = max(a, self.lo) - self.lo, min(b, self.hi) - self.lo
            if b > a:
                total = total + self.g32[a:b].pow(2).sum()
        return total

    # -- update -------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, *, lr_scale: float = 1.0, grad_scale: float = 1.0) -> None:
        self.t += 1
        if grad_scale != 1.0:
            self.g32.mul_(grad_scale)
        lr = self.lr * lr_scale
        cut = min(max(self.n_decayed - self.lo, 0), self.shard)          # [0, cut) decayed, [cut, shard) not
        out = self.flat_p[self.lo:self.hi]
        for a, b, wd in ((0, cut, self.wd), (cut, self.shard, 0.0)):
            if b > a:
                self._adamw(self.master[a:b], self.g32[a:b], self.m[a:b], self.v[a:b], out[a:b], lr, wd)
        if self.world > 1:
            coll.all_gather_into(self.flat_p, out.clone() if dist.get_backend(self.group) != "nccl" else out, self.group)
        self.zero_grad()

    def _adamw(self, p, g, m, v, out, lr, wd):
        b1, b2 = self.betas
        if p.is_cuda and out.dtype == torch.bfloat16 and p.numel() % 4 == 0:
            from .fused import fused_adamw_

            fused_adamw_(p, g, m, v, out, step=self.t, lr=lr, beta1=b1, beta2=b2, eps=self.eps, wd=wd)
            return
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        p.mul_(1 - lr * wd)
        p.addcdiv_(m / (1 - b1 ** self.t), (v / (1 - b2 ** self.t)).sqrt_().add_(self.eps), value=-lr)
        out.copy_(p)

    def state_dict(self) -> dict:
        return {"t": self.t, "master": self.master, "m": self.m, "v": self.v, "rank": self.rank, "world": self.world}

    def load_state_dict(self, sd: dict) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank:
            raise ValueError("optimizer shard belongs to another rank layout")
        self.t = int(sd["t"])
        for k in ("master", "m", "v"):
            getattr(self, k).copy_(sd[k])
