"""Builds the CUDA kernels into ``acache_b200/csrc/libacache_b200.so`` (sm_100a only).

Usage: ``python -m acache_b200.build [--force] [--verbose]``.  Every ``.cu`` under
``csrc/`` is compiled with nvcc to an object file (in parallel) and linked into one
shared library that exports the C ABI of ``include/acache_b200.h``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB = CSRC / "libacache_b200.so"
OBJ = CSRC / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _stamp(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + [CSRC.parents[1] / "include" / "acache_b200.h"]:
        h.update(hdr.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(src: Path):
        obj = OBJ / (src.stem + ".o")
        stamp_file = OBJ / (src.stem + ".stamp")
        stamp = _stamp(src)
        if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
            return obj, False, ""
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        stamp_file.write_text(stamp)
        return obj, True, res.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(compile_one, sources))
    if verbose:
        for (_, _, log), src in zip(results, sources):
            if log:
                print(f"--- {src.name}\n{log}")
    objs = [str(o) for o, _, _ in results]
    rebuilt = any(r for _, r, _ in results)
    if rebuilt or force or not LIB.exists():
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *objs,
               "-Xlinker", "--exclude-libs,ALL"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
