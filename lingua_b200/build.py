"""Builds ``lingua_b200/lib/liblingua_b200.so`` from ``lingua_b200/csrc/*.cu`` with nvcc for sm_100a.

The library has a plain C ABI (no torch headers), so a full rebuild takes well under a
minute and needs no GPU. Objects are cached by a hash of the source, the headers and the
flags. ``python -m lingua_b200.build [--verbose] [--force]``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = LIBDIR / "obj"
LIB = LIBDIR / "liblingua_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
    *os.environ.get("LB_EXTRA_NVCC_FLAGS", "").split(),  # e.g. -DLB_ATTN_TRACE for the timing trace of attention.cu
]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put /usr/local/cuda/bin on PATH")
    return cand


def _digest(src: Path, headers: list[Path]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in [src, *headers]:
        h.update(f.read_bytes())
    return h.hexdigest()[:16]


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    """Compile every kernel source and link the shared library. Returns its path. ``debug_bounds`` builds the
    bounds-checked variant (``-DLB_DEBUG_BOUNDS``, see csrc/common.cuh) next to the regular one as
    ``liblingua_b200_dbg.so``; ``LINGUA_B200_LIB`` selects which file ``ops/_lib.py`` loads."""
    if debug_bounds:
        return _build_variant(["-DLB_DEBUG_BOUNDS"], LIBDIR / "liblingua_b200_dbg.so", LIBDIR / "obj_dbg", verbose)
    nvcc = nvcc_path()
    OBJDIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJDIR / f"{src.stem}.{_digest(src, headers)}.o"
        objs.append(obj)
        if force or not obj.exists():
            for old in OBJDIR.glob(f"{src.stem}.*.o"):
                old.unlink()
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = OBJDIR / f"{src.stem}.ptxas.log"
        log.write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"[build] {src.name}\n{r.stderr}")
        return obj

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not LIB.exists() or force:
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def _build_variant(extra: list, lib: Path, objdir: Path, verbose: bool) -> Path:
    nvcc = nvcc_path()
    objdir.mkdir(parents=True, exist_ok=True)
    objs = []

    def compile_one(src):
        obj = objdir / f"{src.stem}.o"
        r = subprocess.run([nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"[build] {src.name} {' '.join(extra)}")
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, sorted(CSRC.glob("*.cu"))))
    r = subprocess.run([nvcc, "-shared", "-o", str(lib), *map(str, objs), "-lcudart"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, debug_bounds="--debug-bounds" in sys.argv)
    print(p)
