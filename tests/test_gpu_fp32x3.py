"""GPU parity of the FP32X3 variant: float storage, tensor-core tile GEMM on operands split into TF32 head and tail.

Each FP32 product of the transform domain is rebuilt from three TF32 products (hi*hi + lo*hi + hi*lo), so the
variant has to meet the FP32 bar of BASELINE.json's north_star, max|y - ref| / max|ref| <= 1e-4 against the
double-accumulating direct-convolution oracle, and be at least as close to it as the exact FFMA path (to which it
is not bit-identical).
The reference has FP32 FFMA arithmetic only (comparison/GEMM.cuh:124-255), so this variant is pinned by the oracle
and by the golden Conv_<L> fixtures of the reference's numpy model.
"""
import ctypes
import glob
import os
import random

import numpy as np
import pytest

import oracle
from util import LAYOUTS, make_inputs, maxrel, run_conv, to_dev

pytestmark = pytest.mark.gpu
TOL = 1e-4          # the FP32 bar
NEAR_FP32 = 5e-5    # distance to the exact FFMA path of the same Winograd algorithm (whose own error is ~2e-5)
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "conv_*.npz")))


@pytest.fixture(scope="module")
def cb():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import cudnntest_b200
    cudnntest_b200.lib()
    return cudnntest_b200


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_golden_fixtures(cb, path):
    """The reference's own Conv_<L> / Winograd outputs (numpy model) on its seeded inputs."""
    layout = os.path.basename(path).split("_")[1]
    d = np.load(path)
    x, wt = oracle.from_layout(d["x"], layout), oracle.from_layout(d["w"], layout)   # filters permute like activations
    y = run_conv(x, wt, None, layout, dtype="fp32x3", wino=4)
    assert maxrel(y, oracle.from_layout(d["conv"], layout)) <= TOL
    assert maxrel(y, oracle.from_layout(d["wino"], layout)) <= TOL


@pytest.mark.parametrize("m", [4, 2])
@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("shape", [(4, 64, 28, 28, 96), (3, 40, 9, 13, 72), (1, 512, 14, 14, 512), (2, 20, 11, 7, 10),
                                   (2, 264, 8, 8, 264), (1, 8, 1, 1, 8)])
def test_against_oracle_and_exact_path(cb, shape, layout, m):
    """Ragged tiles, channel counts that end inside a 32-float ring slot (40, 20, 264: the slot's remainder holds the
    other half of the row and must not be multiplied), 512-deep contractions (256-filter tiles), fused epilogue."""
    n, c, h, w, k = shape
    pool = h % 2 == 0 and w % 2 == 0
    x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape) + m)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True, pool=pool)
    y = run_conv(x, wt, b, layout, dtype="fp32x3", wino=m, relu=True, pool=pool)
    assert maxrel(y, ref) <= TOL
    y32 = run_conv(x, wt, b, layout, dtype="fp32", wino=m, relu=True, pool=pool)
    assert maxrel(y, y32.astype(np.float64)) <= NEAR_FP32
    assert maxrel(y, ref) <= 1.5 * maxrel(y32, ref) + 2e-6      # at least as close to the oracle as the FFMA path


def test_error_is_fp32_level_not_tf32_level(cb):
    """On a 256-channel layer the split variant is two orders of magnitude closer to the oracle than plain TF32."""
    n, c, h, w, k = 2, 256, 28, 28, 128
    x, wt, b = make_inputs(n, c, h, w, k, seed=77)
    ref = oracle.conv_f64(x, wt, bias=b)
    e3 = maxrel(run_conv(x, wt, b, "NHWC", dtype="fp32x3", wino=4), ref)
    e1 = maxrel(run_conv(x, wt, b, "NHWC", dtype="tf32", wino=4), ref)
    e0 = maxrel(run_conv(x, wt, b, "NHWC", dtype="fp32", wino=4), ref)
    assert e3 <= TOL and e3 <= 4 * e0 + 1e-6 and e3 * 20 <= e1, (e0, e3, e1)


@pytest.mark.parametrize("src", LAYOUTS)
def test_layout_pairs_and_engine_choice(cb, src):
    """wino = 0 (the engine's choice) and every output layout; C <= 3 lands on the exact FFMA direct kernel."""
    for shape in ((2, 24, 10, 12, 40), (2, 3, 16, 16, 64)):
        n, c, h, w, k = shape
        x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape))
        ref = oracle.conv_f64(x, wt, bias=b, relu=True)
        base = run_conv(x, wt, b, src, dtype="fp32x3", relu=True)
        assert maxrel(base, ref) <= TOL
        for dst in LAYOUTS:
            y = run_conv(x, wt, b, src, layout_out=dst, dtype="fp32x3", relu=True)
            assert np.array_equal(y, base)


def test_slab_invariance_is_bitwise(cb):
    n, c, h, w, k = 5, 48, 12, 12, 64
    x, wt, b = make_inputs(n, c, h, w, k, seed=5)
    whole = run_conv(x, wt, b, "NHWC", dtype="fp32x3", wino=4, relu=True)
    for slab in (1, 2, 3):
        assert np.array_equal(run_conv(x, wt, b, "NHWC", dtype="fp32x3", wino=4, relu=True, slab_images=slab), whole)


def test_static_scratch_entry_point(cb):
    """The allocation-free entry point sizes its slabs from the same geometry (rows of 2*Cp floats)."""
    import torch
    n, c, h, w, k = 3, 64, 20, 20, 64
    x, wt, b = make_inputs(n, c, h, w, k, seed=9)
    L = cb.lib()
    d = cb.make_desc(n, c, h, w, k, layout="NHWC", dtype="fp32x3", wino=4, relu=True, bias=True)
    dp = ctypes.byref(d)
    u = torch.empty(L.wino_filter_bytes(dp), dtype=torch.uint8, device="cuda")
    xd, wd, bd = to_dev(oracle.to_layout(x, "NHWC")), to_dev(oracle.filter_to_layout(wt, "NHWC")), to_dev(b)
    y = torch.empty(cb.act_shape("NHWC", n, k, h, w), dtype=torch.float32, device="cuda")
    assert L.wino_filter_transform(dp, wd.data_ptr(), u.data_ptr(), None) == 0
    assert L.wino_conv_forward_static(dp, xd.data_ptr(), u.data_ptr(), bd.data_ptr(), y.data_ptr(), None) == 0
    cb.device_status()
    got = oracle.from_layout(y.cpu().numpy(), "NHWC")
    assert np.array_equal(got, run_conv(x, wt, b, "NHWC", dtype="fp32x3", wino=4, relu=True))


def test_random_shapes(cb):
    rng = random.Random(2024)
    for it in range(30):
        c = rng.choice([1, 3, 8, 24, 40, 64, 100, 136])
        k = rng.choice([8, 16, 48, 64, 80, 130, 256, 272])
        h, w, n = rng.randint(1, 30), rng.randint(1, 30), rng.randint(1, 3)
        pool = rng.random() < 0.4 and h >= 2 and w >= 2
        layout, m = rng.choice(LAYOUTS), rng.choice([0, 2, 4])
        pad = rng.choice([1, 1, 0]) if h >= 3 and w >= 3 else 1
        x, wt, b = make_inputs(n, c, h, w, k, seed=9000 + it)
        ref = oracle.conv_f64(x, wt, bias=b, relu=True, pool=pool, pad=pad)
        if ref.size == 0:
            continue
        y = run_conv(x, wt, b, layout, dtype="fp32x3", wino=m, relu=True, pool=pool, pad=pad)
        assert y.shape == ref.shape
        assert np.abs(y - ref).max() <= TOL * max(np.abs(ref).max(), 1e-30), (layout, m, (n, c, h, w, k), pool, pad)


@pytest.mark.parametrize("shape,layout,m", [((64, 256, 56, 56, 256), "NHWC", 4), ((64, 512, 28, 28, 512), "CHWN", 4),
                                            ((64, 512, 28, 28, 512), "NHWC", 2)])
def test_full_size_configs_properties(cb, shape, layout, m):
    """BASELINE configs 1 and 2 at full size: the first two images against the oracle, the whole batch against itself
    under a different slab size (bitwise), and image independence (permuting the batch permutes the output)."""
    n, c, h, w, k = shape
    x, wt, b = make_inputs(n, c, h, w, k, seed=0xC0DE0010 + m)
    y = run_conv(x, wt, b, layout, dtype="fp32x3", wino=m, relu=True)
    assert np.array_equal(y, run_conv(x, wt, b, layout, dtype="fp32x3", wino=m, relu=True, slab_images=5))
    assert maxrel(y[:2], oracle.conv_f64(x[:2], wt, bias=b, relu=True)) <= TOL
    perm = np.random.default_rng(0).permutation(n)
    assert np.array_equal(run_conv(x[perm], wt, b, layout, dtype="fp32x3", wino=m, relu=True), y[perm])
