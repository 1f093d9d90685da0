"""ctypes binding of the in-tree native library (``libnga_b200.so``).

The library is built by ``archlab_b200/csrc/build.py`` and shares torch's CUDA runtime, so raw
device pointers and the current torch stream are passed straight through.  On a machine with a
GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "libnga_b200.so"
_lib = None
_status = {}

EPI_SCALE, EPI_AXPBY, EPI_RELU2, EPI_MUL_DRELU2, EPI_ATOMIC_ADD = 0, 1, 2, 3, 4


class NativeError(RuntimeError):
    pass


def available() -> bool:
    return torch.cuda.is_available() and _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise NativeError(
                f"{_LIB_PATH} is missing: run `python archlab_b200/csrc/build.py` "
                "(the CUDA path has no PyTorch fallback on a GPU machine)"
            )
        _lib = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    c = ctypes
    vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
    L.nga_gemm_bf16.argtypes = [vp, vp, vp, vp, i, i, i, i, ll, ll, ll, ll, ll, ll, ll, ll,
                                i, i, i, i, i, f, f, i, vp, vp]
    L.nga_gemm_bf16.restype = i
    L.nga_gemm2_bf16.argtypes = L.nga_gemm_bf16.argtypes
    L.nga_gemm2_bf16.restype = i
    L.nga_launch_count.restype = ll
    L.nga_launch_count_reset.restype = None
    for name, sig in _EXTRA_SIGNATURES.items():
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.argtypes, fn.restype = sig


# name -> (argtypes, restype); filled by the op modules before first use of ``lib()``.
_EXTRA_SIGNATURES: dict[str, tuple[list, object]] = {}


def register_signature(name: str, argtypes: list, restype=ctypes.c_int) -> None:
    _EXTRA_SIGNATURES[name] = (argtypes, restype)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes, fn.restype = argtypes, restype


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait gives up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status[key]


def check_status() -> None:
    """Synchronise and raise if any kernel on this device reported a timed-out wait."""
    w = status_word()
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise NativeError(f"device status word = {code} (1 = mbarrier wait timed out, 2 = peer flag wait timed out)")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")


def launch_count() -> int:
    return int(lib().nga_launch_count())


def launch_count_reset() -> None:
    lib().nga_launch_count_reset()
