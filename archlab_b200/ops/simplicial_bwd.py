"""Launcher of the sm_100a 2-simplicial backward (``csrc/simplicial_bwd.cu``): a query-owned kernel
for dq / dk1 / dv1 and a key-owned kernel for dk2 / dv2, both with TMEM-resident accumulators.

``deterministic``: None follows ``torch.are_deterministic_algorithms_enabled()`` (the switch the reference honours,
src/archlab/architectures/simplicial_attention.py:93-94).  The default path adds the short-key gradients (and, under
GQA, the long-key gradients of the heads of a group) with fp32 atomics; the deterministic path stores every
contribution and sums in a fixed order, bit-reproducibly, at the price of ``2 x B*N*w1*Hq*128`` fp32 of scratch."""
from __future__ import annotations

import ctypes as C

import torch

from . import native
from .simplicial_cuda import _rows


native.register_signature("nga_simplicial_bwd_set_deterministic", [C.c_void_p] * 4, None)


def simplicial_bwd(q, k1, k2, v1, v2, out, dout, lse2, w1: int, w2: int, scale: float, deterministic: bool | None = None):
    if deterministic is None:
        deterministic = torch.are_deterministic_algorithms_enabled()
    B, N, Hq, D = q.shape
    Hkv = k1.shape[2]
    (q, ldq), (k1, ldk1), (k2, ldk2), (v1, ldv1), (v2, ldv2), (out, ldo), (dout, lddo) = (
        _rows(t) for t in (q, k1, k2, v1, v2, out, dout))
    dev = q.device
    dq = torch.empty(B, N, Hq, D, dtype=torch.bfloat16, device=dev)
    dk1, dk2, dv1, dv2 = (torch.empty(B, N, Hkv, D, dtype=torch.bfloat16, device=dev) for _ in range(4))
    dk1_acc = torch.empty(B * N, Hkv * D, dtype=torch.float32, device=dev)
    dv1_acc = torch.empty_like(dk1_acc)
    dk2_acc = torch.empty_like(dk1_acc) if Hq != Hkv else None
    dv2_acc = torch.empty_like(dk1_acc) if Hq != Hkv else None
    delta = torch.empty(B, Hq, N, dtype=torch.float32, device=dev)
    if deterministic:
        part = [torch.empty(B * N * w1 * Hq, D, dtype=torch.float32, device=dev) for _ in range(2)]
        planes = [torch.empty(Hq // Hkv, B * N, Hkv * D, dtype=torch.float32, device=dev) if Hq != Hkv else None for _ in range(2)]
        native.lib().nga_simplicial_bwd_set_deterministic(part[0].data_ptr(), part[1].data_ptr(),
                                                         None if planes[0] is None else planes[0].data_ptr(),
                                                         None if planes[1] is None else planes[1].data_ptr())
    rc = native.lib().nga_simplicial_bwd(
        q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(), out.data_ptr(), dout.data_ptr(),
        lse2.data_ptr(), dq.data_ptr(), dk1.data_ptr(), dk2.data_ptr(), dv1.data_ptr(), dv2.data_ptr(),
        dk1_acc.data_ptr(), dv1_acc.data_ptr(), None if dk2_acc is None else dk2_acc.data_ptr(),
        None if dv2_acc is None else dv2_acc.data_ptr(), delta.data_ptr(), ldq, ldk1, ldk2, ldv1, ldv2, ldo, lddo,
        Hq * D, Hkv * D, Hkv * D, Hkv * D, Hkv * D, B, N, Hq, Hkv, D, w1, w2, scale,
        native.status_word(dev).data_ptr(), native.stream_ptr())
    native.check(rc, "nga_simplicial_bwd")
    return dq, dk1, dk2, dv1, dv2
