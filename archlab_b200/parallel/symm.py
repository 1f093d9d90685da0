"""Symmetric (peer-mapped) device memory over NVLink.

A ``SymmTensor`` is a tensor allocated at the same offset on every rank of a process group and
mapped into every process (CUDA VMM handles exchanged once at rendezvous through
``torch.distributed._symmetric_memory``, which is only used here as the allocator / handle
exchange).  Kernels receive the per-rank base addresses and issue ordinary ``ld`` / ``st`` to peers
from inside compute kernels; cross-rank ordering uses ``PeerBarrier`` (flags in symmetric memory,
release / acquire at system scope, bounded wait reporting through the device status word).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import native

# The kernels here use plain peer loads / stores only, so the buffers are not bound to an NVSwitch
# multicast object (a rank that dies while bound can fault its peers' GPUs); opt in by setting the
# variable to 0 before import.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
native.register_signature("nga_peer_barrier", [_vp, _i, _i, _i, _vp, _vp])


@dataclass
class SymmTensor:
    tensor: torch.Tensor            # this rank's buffer
    ptrs: list[int]                 # base address of the same buffer on every rank (index = rank)
    handle: object
    multicast_ptr: int = 0

    def ptr_array(self, elem_offset: int = 0):
        """ctypes array of per-rank addresses of element ``elem_offset``."""
        esz = self.tensor.element_size()
        return (C.c_longlong * len(self.ptrs))(*[p + elem_offset * esz for p in self.ptrs])


def symm_empty(shape, dtype, device, group=None) -> SymmTensor:
    import torch.distributed._symmetric_memory as sm

    group = group or dist.group.WORLD
    t = sm.empty(*shape, dtype=dtype, device=device) if isinstance(shape, (tuple, list)) else sm.empty(
        shape, dtype=dtype, device=device)
    h = sm.rendezvous(t, group)
    ptrs = [int(p) for p in h.buffer_ptrs]
    mc = int(h.multicast_ptr) if getattr(h, "has_multicast_support", lambda *a: False) and h.multicast_ptr else 0
    return SymmTensor(t, ptrs, h, mc)


def symm_zeros(shape, dtype, device, group=None) -> SymmTensor:
    st = symm_empty(shape, dtype, device, group)
    st.tensor.zero_()
    return st


class PeerBarrier:
    """Device-side barrier between the ranks of a group, enqueued on the current stream."""

    def __init__(self, device, group=None):
        self.group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.flags = symm_zeros((64,), torch.int32, device, self.group)
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(self.group)          # flags are zero everywhere before the first device barrier

    def __call__(self) -> None:
        self.epoch += 1
        rc = native.lib().nga_peer_barrier(self.flags.ptr_array(), self.rank, self.world, self.epoch,
                                           native.status_word(self.flags.tensor.device).data_ptr(),
                                           native.stream_ptr())
        native.check(rc, "nga_peer_barrier")
