"""Encoded weights resident in host memory: selected tensors of safetensors shards, bit for bit, behind tensor views.

Serving a large MoE from one box keeps the routed experts' *encoded* weights (int8 payloads, e8m0 / fp8 scales, bf16) in
pinned host memory and moves only what a step needs.  This store reads the tensors chosen by a name predicate straight
from the shard files into one byte buffer per shard: the safetensors header gives every tensor's byte range, adjacent
ranges are merged, and a bounded thread pool fills the buffer with positional reads of at most 32 MiB each.  Nothing is
decoded or converted, so ``get(name)`` is a view with the file's dtype and shape.  Before allocating, the store checks
that the machine has the bytes plus a reserve available and refuses otherwise (the reference keeps its V4.1 experts this
way: src/archlab/automodel/deepseek_v41_cpu_store.py:16-151).
"""
from __future__ import annotations

import concurrent.futures
import json
import math
import os
import struct
import time
from pathlib import Path
from typing import Callable

import torch

DTYPES = {"I8": torch.int8, "U8": torch.uint8, "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I32": torch.int32,
          "I64": torch.int64, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2}
if hasattr(torch, "float8_e8m0fnu"):
    DTYPES["F8_E8M0"] = torch.float8_e8m0fnu
READ_BYTES = 32 * 1024 ** 2


def shard_header(path: Path) -> tuple[int, dict]:
    """(offset of the data section, tensor table) of a safetensors file."""
    with path.open("rb") as f:
        (length,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(length))
    header.pop("__metadata__", None)
    return 8 + length, header


def available_bytes() -> int:
    for line in Path("/proc/meminfo").read_text().splitlines():
        if line.startswith("MemAvailable:"):
            return int(line.split()[1]) * 1024
    raise OSError("MemAvailable is not reported")


class ResidentTensorStore:
    def __init__(self, root, select: Callable[[str], bool], *, threads: int = 8, pinned: bool = True, reserve_bytes: int = 64 * 2 ** 30,
                 log=None):
        t0 = time.monotonic()
        root = Path(root)
        weight_map = json.loads((root / "model.safetensors.index.json").read_text())["weight_map"]
        shards = sorted({file for name, file in weight_map.items() if select(name)})
        plans, total = [], 0
        for file in shards:
            if Path(file).name != file:
                raise ValueError("shard escapes the model directory")
            data_start, table = shard_header(root / file)
            chosen = sorted(((n, m) for n, m in table.items() if select(n)), key=lambda nm: nm[1]["data_offsets"][0])
            size = sum(m["data_offsets"][1] - m["data_offsets"][0] for _, m in chosen)
            plans.append((root / file, data_start, chosen, size))
            total += size
        have = available_bytes()
        if total + reserve_bytes > have:
            raise MemoryError(f"the store needs {total / 2 ** 30:.1f} GiB plus a reserve of {reserve_bytes / 2 ** 30:.1f} GiB; "
                              f"{have / 2 ** 30:.1f} GiB are available")
        self.entries: dict[str, torch.Tensor] = {}
        self.buffers, work = [], []
        for path, data_start, chosen, size in plans:
            file_size = path.stat().st_size
            buffer = torch.empty(size, dtype=torch.uint8, pin_memory=pinned and torch.cuda.is_available())
            self.buffers.append(buffer)
            raw = memoryview(buffer.numpy())
            at, ranges = 0, []
            for name, meta in chosen:
                lo, hi = meta["data_offsets"]
                dtype = DTYPES.get(meta["dtype"])
                if dtype is None or hi - lo != math.prod(meta["shape"]) * torch.empty((), dtype=dtype).element_size():
                    raise ValueError(f"unexpected encoding or extent: {name}")
                if data_start + hi > file_size:
                    raise ValueError(f"tensor exceeds its shard: {name}")
                self.entries[name] = buffer.narrow(0, at, hi - lo).view(dtype).reshape(meta["shape"])
                if ranges and ranges[-1][0] + ranges[-1][2] == data_start + lo and ranges[-1][1] + ranges[-1][2] == at:
                    ranges[-1] = (ranges[-1][0], ranges[-1][1], ranges[-1][2] + hi - lo)       # adjacent in file and buffer
                else:
                    ranges.append((data_start + lo, at, hi - lo))
                at += hi - lo
            for src, dst, count in ranges:
                work += [(path, src + off, raw[dst + off:dst + off + min(READ_BYTES, count - off)]) for off in range(0, count, READ_BYTES)]

        def read(item) -> int:
            path, offset, target = item
            fd, done = os.open(path, os.O_RDONLY), 0
            try:
                while done < len(target):
                    n = os.preadv(fd, [target[done:]], offset + done)
                    if n <= 0:
                        raise OSError(f"short read: {path}:{offset + done}")
                    done += n
            finally:
                os.close(fd)
            return done

        with concurrent.futures.ThreadPoolExecutor(max(1, threads)) as pool:
            copied = sum(pool.map(read, work))
        if copied != total:
            raise RuntimeError("incomplete host store")
        self.report = {"bytes": total, "tensors": len(self.entries), "shards": len(plans), "reads": len(work), "threads": threads,
                       "pinned": bool(self.buffers and self.buffers[0].is_pinned()), "seconds": time.monotonic() - t0, "encoding_unchanged": True}
        if log is not None:
            log(json.dumps({"event": "host_store_ready", **self.report}))

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def get(self, name: str) -> torch.Tensor:
        return self.entries[name]

    def to_device(self, names, device, *, non_blocking: bool = True) -> dict[str, torch.Tensor]:
        """Copies of the named tensors on ``device`` (asynchronous from pinned memory)."""
        return {n: self.entries[n].to(device, non_blocking=non_blocking) for n in names}
