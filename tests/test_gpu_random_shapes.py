"""Seeded random shapes through the engine's own choice of kernel (wino = 0), against the direct-convolution oracle.

Every dtype, layout, ragged image size, filter count that fills its last block only partly, optional bias / ReLU /
pool / padding: the shapes land on the thin-input kernels, the three direct tensor-core kernels (with the NHWC
staging route for NCHW / CHWN) and the Winograd pipeline alike.  Tolerances as everywhere: FP32 max|d| / max|ref|
<= 1e-4, TF32 / BF16 relative L2 <= 5e-3."""
import random

import numpy as np
import pytest

import oracle
from util import make_inputs, rel_l2, run_conv

pytestmark = pytest.mark.gpu


def _case(rng, it):
    dtype = rng.choice(["bf16", "bf16", "tf32", "fp32"])
    if dtype == "bf16":
        c = rng.choice([64, 128, 192, 256, 320, 512])
    elif dtype == "tf32":
        c = rng.choice([3, 32, 64, 96, 128, 256])
    else:
        c = rng.choice([1, 3, 8, 24, 40])
    k = rng.choice([16, 48, 64, 80, 128, 144, 256, 272, 384, 512, 640])
    h, w = rng.randint(1, 36), rng.randint(1, 36)
    n = rng.randint(1, 3)
    pool = rng.random() < 0.4 and h >= 2 and w >= 2
    layout = rng.choice(["NHWC", "NHWC", "NCHW", "CHWN"])
    relu, bias = rng.random() < 0.7, rng.random() < 0.7
    pad = rng.choice([1, 1, 1, 0]) if h >= 3 and w >= 3 else 1
    return dtype, layout, n, c, h, w, k, pool, relu, bias, pad


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes(seed):
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    rng = random.Random(seed)
    for it in range(40):
        dtype, layout, n, c, h, w, k, pool, relu, bias, pad = _case(rng, it)
        x, wt, b = make_inputs(n, c, h, w, k, seed=1000 * seed + it)
        if not bias:
            b = None
        ref = oracle.conv_f64(x, wt, bias=b, relu=relu, pool=pool, pad=pad)
        if ref.size == 0:
            continue
        y = run_conv(x, wt, b, layout, dtype=dtype, relu=relu, pool=pool, pad=pad)
        what = (dtype, layout, (n, c, h, w, k), pool, relu, bias, pad)
        assert y.shape == ref.shape, what
        if dtype == "fp32":
            assert np.abs(y - ref).max() <= 1e-4 * max(np.abs(ref).max(), 1e-30), what
        elif np.abs(ref).max() > 0:
            assert rel_l2(y, ref) <= 5e-3, what
        else:
            assert np.abs(y).max() == 0, what
