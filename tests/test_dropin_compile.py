"""The drop-in claim, literally: the reference's own per-layer benchmark host, comparison/layoutCompare.cu, compiles
unchanged for sm_100a when "DataLayoutTrans.cuh" and "wrapedConv_CuDNN.cuh" resolve to this library's headers
(include/wino_compat.cuh, include/wino_cudnn_compat.cuh) instead of the reference's kernels.

The reference checkout is not part of this repository: the test looks for it in $CUDNNTEST_REFERENCE_DIR or in a
directory named `reference` beside the repository, and is skipped when there is none.  The reference file is copied
to a temporary directory for the compile only; its helper headers util.h and error_util.h (file IO and NVIDIA's
sample macros, which a maintainer keeps) are found through -I.
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_dir():
    for cand in (os.environ.get("CUDNNTEST_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "comparison", "layoutCompare.cu")):
            return cand
    return None


def test_reference_layout_compare_compiles_against_the_shims(tmp_path):
    ref = _reference_dir()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if ref is None or not os.path.exists(nvcc):
        pytest.skip("no reference checkout (or no nvcc) on this machine")
    shutil.copy(os.path.join(ref, "comparison", "layoutCompare.cu"), tmp_path / "layoutCompare.cu")
    (tmp_path / "DataLayoutTrans.cuh").write_text('#pragma once\n#include "wino_compat.cuh"\n')
    (tmp_path / "wrapedConv_CuDNN.cuh").write_text('#pragma once\n#include "wino_cudnn_compat.cuh"\n')
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-c", "layoutCompare.cu", "-o", "layoutCompare.o",
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ref, "comparison")]
    r = subprocess.run(cmd, cwd=tmp_path, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    # and it links against libwino + cuDNN: every symbol the reference host needs is there
    so_dir = os.path.join(ROOT, "cudnntest_b200")
    if os.path.exists(os.path.join(so_dir, "libwino.so")):
        r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "layoutCompare.o", "-o", "layoutCompare",
                            "-L", so_dir, "-lwino", "-lcudnn"], cwd=tmp_path, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-3000:]
