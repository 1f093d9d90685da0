"""Deterministic raw-int32 token batches with data-parallel prefix ownership
(src/archlab/megatron/token_batches.py:12-136).

Batch ``b`` reads part ``b mod P`` at flat token offset ``(b div P) * batch * seq`` (cyclic),
``batch*seq + 1`` tokens; labels are the tokens shifted by one.  Data ownership depends on the
DATA-PARALLEL rank only, so tensor / pipeline / expert / context ranks of one replica read identical
batches.  ``NativeTokenBatches`` is the same iterator backed by the C++ prefetching reader
(``csrc/token_reader.cu``).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np
import torch


def partition_prefixes(prefixes: list[Path], rank: int, world_size: int, *, require_distinct: bool = True) -> list[Path]:
    if not prefixes:
        raise ValueError("at least one indexed-data prefix is required")
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"invalid rank/world size: {rank}/{world_size}")
    if require_distinct and len(prefixes) < world_size:
        raise ValueError("training requires at least one distinct indexed-data part per rank: "
                         f"parts={len(prefixes)}, world_size={world_size}")
    return prefixes[rank::world_size] or [prefixes[rank % len(prefixes)]]


partition_prefixes_for_dp_rank = partition_prefixes


class BinaryTokenBatches:
    def __init__(self, prefixes, *, batch_size: int, sequence_len: int, start_batch: int, device,
                 repeat_window_batches: int | None = None):
        if not prefixes:
            raise ValueError("at least one indexed-data prefix is required")
        self.arrays = [np.memmap(f"{p}.bin", mode="r", dtype=np.int32) for p in prefixes]
        if any(a.size <= sequence_len for a in self.arrays):
            raise ValueError("each indexed-data part must contain more than one sequence")
        if repeat_window_batches is not None and repeat_window_batches < 1:
            raise ValueError("repeat_window_batches must be positive")
        self.batch_size, self.sequence_len = batch_size, sequence_len
        self.batch_index = self.start_batch = start_batch
        self.repeat_window_batches = repeat_window_batches
        self.device = torch.device(device)

    @staticmethod
    def _cyclic_slice(array, start: int, length: int) -> np.ndarray:
        start %= array.size
        idx = (start + np.arange(length)) % array.size
        return np.asarray(array[idx]) if start + length > array.size else np.asarray(array[start:start + length])

    def _source_index(self, b: int) -> int:
        if self.repeat_window_batches is None:
            return b
        return self.start_batch + (b - self.start_batch) % self.repeat_window_batches

    def cpu_block(self, batch_index: int) -> torch.Tensor:
        src = self._source_index(batch_index)
        array = self.arrays[src % len(self.arrays)]
        flat = self.batch_size * self.sequence_len
        window = self._cyclic_slice(array, (src // len(self.arrays)) * flat, flat + 1)
        return torch.from_numpy(np.array(window, dtype=np.int64, copy=True))

    def __iter__(self):
        return self

    def __next__(self) -> dict[str, torch.Tensor]:
        t = self.cpu_block(self.batch_index)
        self.batch_index += 1
        if self.device.type == "cuda":
            t = t.pin_memory()
        x = t[:-1].view(self.batch_size, self.sequence_len)
        y = t[1:].view(self.batch_size, self.sequence_len)
        return {"tokens": x.to(self.device, non_blocking=True), "labels": y.to(self.device, non_blocking=True)}


DPRankTokenBatches = BinaryTokenBatches


class NativeTokenBatches:
    """Same batches as ``BinaryTokenBatches``; reading and int32->int64 widening run one batch
    ahead in a native worker thread and land in a reusable pinned buffer."""

    def __init__(self, prefixes, *, batch_size: int, sequence_len: int, start_batch: int, device,
                 repeat_window_batches: int | None = None):
        from ..ops import native

        L = native.lib()
        L.nga_reader_open.argtypes = [C.POINTER(C.c_char_p), C.c_int, C.c_longlong, C.c_longlong, C.c_longlong,
                                      C.c_longlong]
        L.nga_reader_open.restype = C.c_void_p
        L.nga_reader_next.argtypes = [C.c_void_p, C.c_void_p]
        L.nga_reader_next.restype = C.c_longlong
        L.nga_reader_close.argtypes = [C.c_void_p]
        L.nga_reader_close.restype = None
        self._L = L
        paths = [str(Path(f"{p}.bin")).encode() for p in prefixes]
        arr = (C.c_char_p * len(paths))(*paths)
        self.batch_size, self.sequence_len = batch_size, sequence_len
        self.device = torch.device(device)
        self._h = L.nga_reader_open(arr, len(paths), batch_size, sequence_len, start_batch,
                                    repeat_window_batches or 0)
        if not self._h:
            raise ValueError("could not open the indexed-data parts (missing file or shorter than one sequence)")
        n = batch_size * sequence_len + 1
        self._buf = torch.empty(n, dtype=torch.int64, pin_memory=self.device.type == "cuda")
        self.batch_index = start_batch

    def __iter__(self):
        return self

    def __next__(self) -> dict[str, torch.Tensor]:
        self.batch_index = int(self._L.nga_reader_next(self._h, self._buf.data_ptr())) + 1
        t = self._buf
        x = t[:-1].view(self.batch_size, self.sequence_len).to(self.device, non_blocking=True)
        y = t[1:].view(self.batch_size, self.sequence_len).to(self.device, non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()     # the pinned buffer is reused by the next call
        else:
            x, y = x.clone(), y.clone()
        return {"tokens": x, "labels": y}

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._L.nga_reader_close(self._h)
            self._h = None

    def __del__(self):
        self.close()
