"""The allocation-free attention backward (fixed in-module scratch) against the regular entry point."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, T, Hq, Hkv, seed):
    from archlab_b200.ops import trunk
    g = torch.Generator(device="cuda").manual_seed(seed)
    D = 128
    qkv = (torch.randn(B * T, (Hq + 2 * Hkv) * D, device="cuda", generator=g) * 0.5).bfloat16()
    dout = (torch.randn(B * T, Hq * D, device="cuda", generator=g) * 0.1).bfloat16()
    out, lse2 = trunk.attn_fwd(qkv, B, T, Hq, Hkv, D, -1)
    return qkv, out, dout, lse2


def _static_bwd(qkv, out, dout, lse2, B, T, Hq, Hkv, window):
    from archlab_b200.ops import native
    L = native.lib()
    fn = L.nga_attn_bwd_static
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, f, vp, vp]
    fn.restype = ctypes.c_int
    dqkv = torch.empty_like(qkv)
    rc = fn(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse2.data_ptr(), dqkv.data_ptr(), B, T, Hq, Hkv, 128,
            window, 1.0 / math.sqrt(128), native.status_word(qkv.device).data_ptr(), native.stream_ptr())
    return rc, dqkv


def test_static_scratch_matches_regular_entry_twice():
    from archlab_b200.ops import native, trunk
    for n, (B, T, Hq, Hkv) in enumerate([(2, 512, 4, 2), (1, 1024, 3, 3)]):
        qkv, out, dout, lse2 = _case(B, T, Hq, Hkv, seed=n)
        want = trunk.attn_bwd(qkv, out, dout, lse2, B, T, Hq, Hkv, 128, -1).float()
        for _ in range(2):
            rc, got = _static_bwd(qkv, out, dout, lse2, B, T, Hq, Hkv, -1)
            assert rc == 0
            torch.cuda.synchronize()
            native.check_status()
            assert ((got.float() - want).norm() / want.norm()).item() < 8e-3


def test_static_scratch_rejects_oversize():
    from archlab_b200.ops import native
    L = native.lib()
    L.nga_attn_bwd_static_max_elems.restype = ctypes.c_longlong
    limit = L.nga_attn_bwd_static_max_elems()
    B, T, Hq, Hkv = 1, 128, 1, 1
    qkv, out, dout, lse2 = _case(B, T, Hq, Hkv, seed=9)
    big_T = limit // 128 + 128                       # one head: B*T*Hq*128 just above the limit
    rc, _ = _static_bwd(qkv, out, dout, lse2, 1, int(big_T), 1, 1, -1)   # rejected before any launch
    assert rc == -20
