"""Build the native sm_100a library in-tree: every ``*.cu`` in this folder -> ``libnga_b200.so``.

``nvcc`` cross-compiles without a GPU.  Objects are rebuilt only when a source or header is newer.
Files named ``*_mc.cu`` hold kernels that single-GPU runs alone may use and are linked into a
separate ``libnga_b200_1gpu.so`` so the main library never depends on them.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE.parent / "libnga_b200.so"
OBJ = HERE / "build"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _stale(obj: Path, deps: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = sorted(HERE.glob("*.h")) + sorted(HERE.glob("*.cuh"))
    sources = sorted(HERE.glob("*.cu"))
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if _stale(obj, [src, *headers]):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ / (src.stem + ".ptxas.log")).write_text(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stderr[-4000:]}")
        if verbose:
            print(f"compiled {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(compile_one, jobs))
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if jobs or not OUT.exists():
        cmd = [NVCC, "-shared", "-o", str(OUT), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
    return OUT


if __name__ == "__main__":
    print(build(verbose=True))
