"""The kernel sources cross-compile for sm_100a without a GPU, also in the bounds-checked variant."""
import shutil
import subprocess
from pathlib import Path

import pytest

from lingua_b200 import build as B


@pytest.mark.skipif(shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists(), reason="needs nvcc")
def test_bounds_checked_variant_of_the_fused_collective_gemm_compiles(tmp_path):
    """-DLB_DEBUG_BOUNDS turns on the validation of table-driven indices (owner, destination row, block to pull) in
    the kernels that store into or read from peers' memory; the variant has to keep compiling."""
    src = B.CSRC / "gemm2.cu"
    cmd = [B.nvcc_path(), *[f for f in B.NVCC_FLAGS if f not in ("-Xptxas", "-v")], "-DLB_DEBUG_BOUNDS", "-I", str(B.CSRC),
           "-c", str(src), "-o", str(tmp_path / "gemm2_dbg.o")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert (tmp_path / "gemm2_dbg.o").stat().st_size > 0
