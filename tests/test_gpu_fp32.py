"""GPU parity of the exact-FP32 path (FFMA tile GEMM), through the C ABI.

Tolerance: max|y - ref| / max|ref| <= 1e-4 against the double-accumulating direct-convolution oracle
(the bar BASELINE.json's north_star states for the FP32 path).  Relayout and pooling are bit exact.
"""
import ctypes
import glob
import os

import numpy as np
import pytest

import oracle
from util import LAYOUTS, make_inputs, maxrel, rel_l2, run_conv, to_dev

pytestmark = pytest.mark.gpu
TOL = 1e-4
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "conv_*.npz")))


@pytest.fixture(scope="module")
def cb():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import cudnntest_b200
    cudnntest_b200.lib()
    return cudnntest_b200


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_reference_wrappers_on_golden_fixtures(cb, path):
    """wrapedConv_<L> with the reference's calling convention against the reference's own Conv_<L> output."""
    import torch
    layout = os.path.basename(path).split("_")[1]
    d = np.load(path)
    x, w = d["x"], d["w"]
    n, c, h, _ = oracle.from_layout(x, layout).shape
    k = d["conv"].shape[{"NCHW": 1, "NHWC": 3, "CHWN": 0}[layout]]
    sizes = cb.legacy_workspace_floats(n, h, c, k, 1)
    v, u, m = (torch.empty(s, dtype=torch.float32, device="cuda") for s in sizes)
    y = torch.zeros(d["conv"].shape, dtype=torch.float32, device="cuda")
    fn = getattr(cb, "wrapedConv_" + layout)
    chn = fn(n, h, c, k, 1, to_dev(x), to_dev(w), v, u, m, y)
    assert chn == k
    assert maxrel(y.cpu().numpy(), d["conv"]) <= TOL
    assert maxrel(y.cpu().numpy(), d["wino"]) <= TOL


@pytest.mark.parametrize("m", [4, 2])
@pytest.mark.parametrize("layout", LAYOUTS)
def test_stages_against_stage_oracle(cb, layout, m):
    """U, V, M and Y of the four-kernel pipeline, each against the numpy stage model."""
    import torch
    n, c, h, w, k = 3, 20, 13, 10, 12      # c not a multiple of 8, ragged tiles in both directions
    x, wt, b = make_inputs(n, c, h, w, k, seed=100 + m)
    L = cb.lib()
    d = cb.make_desc(n, c, h, w, k, layout=layout, dtype="fp32", wino=m, relu=True, bias=True)
    dp = ctypes.byref(d)
    cp, kq, tp = L.wino_stage_cp(dp), L.wino_stage_kq(dp), L.wino_stage_tile_rows(dp, n)
    a = m + 2
    bny, bnx = oracle.tiles_per_side(h, 1, m), oracle.tiles_per_side(w, 1, m)
    t = n * bny * bnx
    assert tp % 128 == 0 and tp >= t and cp % 8 == 0 and cp >= c
    xd, wd = to_dev(oracle.to_layout(x, layout)), to_dev(oracle.filter_to_layout(wt, layout))
    u = torch.full((a * a, k, cp), float("nan"), device="cuda")
    v = torch.full((a * a, tp, cp), float("nan"), device="cuda")
    mm = torch.full((a * a, tp, kq), float("nan"), device="cuda")
    y = torch.full(cb.act_shape(layout, n, k, h, w), float("nan"), device="cuda")
    P = lambda z: ctypes.c_void_p(z.data_ptr())
    cb._lib.check(L.wino_filter_transform(dp, P(wd), P(u), None))
    cb._lib.check(L.wino_stage_input_transform(dp, P(xd), 0, n, P(v), None))
    cb._lib.check(L.wino_stage_gemm(dp, P(v), P(u), P(mm), n, None))
    cb._lib.check(L.wino_stage_output_transform(dp, P(mm), P(to_dev(b)), P(y), 0, n, None))
    cb.device_status()
    ru = oracle.filter_transform(wt, m)
    rv = oracle.input_transform(x, 1, m, order="image")
    rm = oracle.tile_gemm(rv, ru)
    ry = oracle.output_transform(rm, n, h, w, 1, m, bias=b, relu=True)
    un, vn, mn = u.cpu().numpy(), v.cpu().numpy(), mm.cpu().numpy()
    assert maxrel(un[:, :, :c], ru) <= 1e-5
    assert np.all(un[:, :, c:] == 0), "channel padding of U must be zero"
    assert maxrel(vn[:, :t, :c], rv) <= 1e-5
    assert np.all(vn[:, :t, c:] == 0), "channel padding of V must be zero"
    assert maxrel(mn[:, :t, :k], rm) <= 1e-5
    assert maxrel(oracle.from_layout(y.cpu().numpy(), layout), ry) <= TOL


def test_config0_nchw(cb):
    """BASELINE config 0: N=8, C=K=64, 56x56, NCHW, FP32, no bias/ReLU."""
    x, wt, _ = make_inputs(8, 64, 56, 56, 64, seed=0xC0DE0000, bias=False)
    y = run_conv(x, wt, None, "NCHW")
    ref = oracle.conv_f64(x, wt)
    assert maxrel(y, ref) <= TOL
    assert rel_l2(y, ref) <= 1e-5


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("shape", [(1, 3, 7, 7, 4), (2, 8, 6, 6, 64), (5, 16, 14, 14, 130), (1, 1, 1, 1, 1), (2, 33, 9, 17, 40)])
def test_ragged_shapes(cb, layout, shape):
    """N=1, C=3, K<128, K not a multiple of 4, H not a multiple of 4 or 2, rectangular, 1x1 image."""
    n, c, h, w, k = shape
    x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape))
    for m in (4, 2):
        y = run_conv(x, wt, b, layout, wino=m, relu=True)
        assert maxrel(y, oracle.conv_f64(x, wt, bias=b, relu=True)) <= TOL


@pytest.mark.parametrize("src", LAYOUTS)
@pytest.mark.parametrize("dst", LAYOUTS)
def test_cross_layout_conv(cb, src, dst):
    """The nine (source, destination) layout pairs: wrapedConv_* and convLayoutTrans_*_to_*."""
    import torch
    n, c, h, k = 3, 16, 12, 24
    x, wt, _ = make_inputs(n, c, h, h, k, seed=17, bias=False)
    sizes = cb.legacy_workspace_floats(n, h, c, k, 1)
    v, u, m = (torch.empty(s, dtype=torch.float32, device="cuda") for s in sizes)
    y = torch.zeros(cb.act_shape(dst, n, k, h, h), dtype=torch.float32, device="cuda")
    name = "wrapedConv_" + src if src == dst else "convLayoutTrans_%s_to_%s" % (src, dst)
    chn = getattr(cb, name)(n, h, c, k, 1, to_dev(oracle.to_layout(x, src)), to_dev(oracle.filter_to_layout(wt, src)),
                            v, u, m, y)
    assert chn == k
    assert maxrel(oracle.from_layout(y.cpu().numpy(), dst), oracle.conv_f64(x, wt)) <= TOL


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("m", [4, 2])
def test_fused_epilogue(cb, layout, m):
    """bias + ReLU + 2x2 max-pool fused into the output transform, even and odd sizes."""
    for (h, w) in ((12, 8), (9, 11)):
        x, wt, b = make_inputs(2, 8, h, w, 40, seed=h * w)
        y = run_conv(x, wt, b, layout, wino=m, relu=True, pool=True)
        ref = oracle.conv_f64(x, wt, bias=b, relu=True, pool=True)
        assert y.shape == ref.shape
        assert maxrel(y, ref) <= TOL


def test_slabs_do_not_change_results(cb):
    """Processing the batch in slabs of 1, 3 or all images gives bitwise identical outputs."""
    x, wt, b = make_inputs(7, 16, 10, 10, 16, seed=5)
    ys = [run_conv(x, wt, b, "NHWC", relu=True, slab_images=s) for s in (1, 3, 7)]
    assert np.array_equal(ys[0], ys[1]) and np.array_equal(ys[0], ys[2])
    assert maxrel(ys[0], oracle.conv_f64(x, wt, bias=b, relu=True)) <= TOL


def test_padding_zero(cb):
    x, wt, _ = make_inputs(2, 8, 10, 12, 8, seed=3, bias=False)
    for layout in LAYOUTS:
        y = run_conv(x, wt, None, layout, pad=0)
        assert y.shape == (2, 8, 8, 10)
        assert maxrel(y, oracle.conv_f64(x, wt, pad=0)) <= TOL


@pytest.mark.parametrize("src", LAYOUTS)
@pytest.mark.parametrize("dst", LAYOUTS)
def test_relayout_bit_exact(cb, src, dst):
    import torch
    rng = np.random.default_rng(1)
    # odd extents (scalar path), even ones (paired path), multiples of 8 (16-byte vector path, ragged 64 x 64 tiles)
    for (n, c, h, w) in ((3, 37, 9, 13), (8, 72, 10, 14), (2, 130, 6, 66), (8, 72, 8, 20), (16, 136, 12, 12)):
        x = rng.standard_normal((n, c, h, w)).astype(np.float32)
        for tdt in (torch.float32, torch.bfloat16):
            xs = to_dev(oracle.to_layout(x, src), tdt)
            out = cb.layout_convert(xs, src, dst, n, c, h, w)
            ref = xs.float().cpu().numpy()
            assert np.array_equal(oracle.from_layout(out.float().cpu().numpy(), dst), oracle.from_layout(ref, src))


@pytest.mark.parametrize("layout", LAYOUTS)
def test_maxpool_bit_exact(cb, layout):
    import torch
    for (n, c, h, w) in ((2, 19, 10, 14), (8, 24, 9, 11), (16, 64, 12, 6), (2, 5, 7, 32)):       # scalar and 16-byte-vector paths, odd H / W
        x = np.random.default_rng(2).standard_normal((n, c, h, w)).astype(np.float32)
        for tdt in (torch.float32, torch.bfloat16):
            xs = to_dev(oracle.to_layout(x, layout), tdt)
            out = cb.maxpool2x2(xs, layout, n, c, h, w)
            ref = oracle.maxpool2x2(xs.float().cpu().numpy(), layout)
            assert np.array_equal(out.float().cpu().numpy(), ref)


def test_errors_are_reported(cb):
    """Bad arguments come back as status codes with a message, never as a crash."""
    import torch
    with pytest.raises(cb.WinoError):
        cb.WinoConv(1, 8, 8, 8, 8, pad=3)
    conv = cb.WinoConv(1, 8, 8, 8, 8, layout="NHWC")
    d = conv.desc
    L = cb.lib()
    x = torch.zeros(1, 8, 8, 8, device="cuda")
    rc = L.wino_conv_forward(ctypes.byref(d), x.data_ptr(), conv.u.data_ptr(), None, x.data_ptr(), conv.workspace.data_ptr(), 16, None)
    assert rc == cb._lib.E_WORKSPACE and b"workspace" in L.wino_last_error_string()
    assert L.wino_device_status() == 0


def test_full_size_config1_properties(cb):
    """BASELINE config 1 at full size (N=64, C=K=256, 56x56, NHWC, bias+ReLU): the first two images against
    the oracle, and the whole batch against itself under a different slab size (bitwise)."""
    import torch
    n, c, h, k = 64, 256, 56, 256
    x, wt, b = make_inputs(n, c, h, h, k, seed=0xC0DE0010)
    y = run_conv(x, wt, b, "NHWC", relu=True)
    y2 = run_conv(x, wt, b, "NHWC", relu=True, slab_images=5)
    assert np.array_equal(y, y2)
    ref = oracle.conv_f64(x[:2], wt, bias=b, relu=True)
    assert maxrel(y[:2], ref) <= TOL
    # image independence: permuting the batch permutes the output
    perm = np.random.default_rng(0).permutation(n)
    y3 = run_conv(x[perm], wt, b, "NHWC", relu=True)
    assert np.array_equal(y3, y[perm])
