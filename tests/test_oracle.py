"""The CPU oracle against the reference's own Python model (fixtures in tests/golden/).

The fixtures are outputs of Conv_<L>, ConvAdd_<L> and the Wino_* stage chain of
layoutTest/<L>/data/WinoTran_<L>.py on seeded inputs (tests/golden/make_golden.py).
"""
import glob
import os

import numpy as np
import pytest

import oracle

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "conv_*.npz")))


def _case(path):
    name = os.path.basename(path)[:-4]
    _, layout, tag = name.split("_")
    return layout, tag, np.load(path)


def test_fixtures_present():
    assert len(GOLDEN) == 12


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_direct_conv_matches_reference_python(path):
    layout, _, d = _case(path)
    pad = int(d["pad"])
    y64 = oracle.conv_f64(d["x"], d["w"], pad=pad, layout=layout)
    y32 = oracle.conv_f32(d["x"], d["w"], pad=pad, layout=layout)
    y32p = oracle.conv_f32_plain(d["x"], d["w"], pad=pad, layout=layout)
    ref = d["conv"]
    assert y64.shape == ref.shape
    scale = np.abs(ref).max()
    # Conv_<L> sums in float32 (np.sum of float32 products): agreement to float32 rounding
    assert np.abs(y64 - ref).max() <= 1e-5 * scale
    assert np.abs(y32 - ref).max() <= 1e-5 * scale
    assert np.abs(y32p - ref).max() <= 1e-5 * scale
    if "bias" in d.files:
        yb = oracle.conv_f64(d["x"], d["w"], bias=d["bias"], pad=pad, layout=layout)
        assert np.abs(yb - d["conv_bias"]).max() <= 1e-5 * np.abs(d["conv_bias"]).max()


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_winograd_stages_match_reference_python(path):
    layout, _, d = _case(path)
    pad = int(d["pad"])
    x = oracle.from_layout(d["x"], layout)
    w = oracle.from_layout(d["w"], layout)       # filters permute exactly like activations
    n, c, h, _ = x.shape
    k = w.shape[0]
    bn = oracle.tiles_per_side(h, pad, 4)
    t = n * bn * bn
    v = oracle.input_transform(x, pad, 4, order="ref")
    u = oracle.filter_transform(w, 4)
    m = oracle.tile_gemm(v, u)
    # reference buffers: NHWC V[36][Mp][Kp], U[36][Np][Kp]; NCHW/CHWN V[36][Kp][Mp], U[36][Kp][Np]; M[36][Mp][Np]
    if layout == "NHWC":
        rv, ru = d["V"][:, :t, :c], d["U"][:, :k, :c]
    else:
        rv, ru = d["V"][:, :c, :t].transpose(0, 2, 1), d["U"][:, :c, :k].transpose(0, 2, 1)
    rm = d["M"][:, :t, :k]
    assert np.abs(v - rv).max() <= 1e-5 * np.abs(rv).max()
    assert np.abs(u - ru).max() <= 1e-5 * np.abs(ru).max()
    assert np.abs(m - rm).max() <= 1e-5 * np.abs(rm).max()
    # everything outside the cropped part of the reference buffers is zero padding
    assert np.count_nonzero(d["M"]) <= t * k * 36
    y = oracle.output_transform(m, n, h, h, pad, 4, order="ref")
    ry = oracle.from_layout(d["wino"], layout)
    assert np.abs(y - ry).max() <= 1e-5 * np.abs(ry).max()


@pytest.mark.parametrize("m", [2, 4])
@pytest.mark.parametrize("shape", [(2, 5, 7, 6, 9), (1, 3, 4, 7, 7), (3, 8, 8, 12, 4)])
def test_stage_chain_equals_direct(m, shape):
    """F(2,3) has no pin in the reference: pin it (and rectangular images) to the direct oracle."""
    n, c, k, h, w = shape
    rng = np.random.default_rng(7 + m)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((k, c, 3, 3)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
    b = (rng.standard_normal(k) * 0.01).astype(np.float32)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True)
    for order in ("image", "ref"):
        v = oracle.input_transform(x, 1, m, order=order)
        u = oracle.filter_transform(wt, m)
        y = oracle.output_transform(oracle.tile_gemm(v, u), n, h, w, 1, m, order=order, bias=b, relu=True)
        assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()


def test_layouts_and_epilogue_agree():
    rng = np.random.default_rng(11)
    n, c, k, h, w = 2, 6, 5, 8, 6
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    wt = rng.standard_normal((k, c, 3, 3)).astype(np.float32)
    b = rng.standard_normal(k).astype(np.float32)
    base = oracle.conv_f64(x, wt, bias=b, relu=True, pool=True)
    assert base.shape == (n, k, h // 2, w // 2)
    full = oracle.conv_f64(x, wt, bias=b, relu=True)
    assert np.array_equal(oracle.maxpool2x2(full), base)
    assert (base >= 0).all()
    for li in ("NHWC", "CHWN"):
        for lo in ("NCHW", "NHWC", "CHWN"):
            y = oracle.conv_f64(oracle.to_layout(x, li), oracle.filter_to_layout(wt, li), bias=b, relu=True,
                                pool=True, layout=li, layout_out=lo)
            assert np.array_equal(oracle.from_layout(y, lo), base)
            yf = oracle.conv_f32(oracle.to_layout(x, li), oracle.filter_to_layout(wt, li), bias=b, relu=True,
                                 pool=True, layout=li, layout_out=lo)
            assert np.abs(oracle.from_layout(yf, lo) - base).max() <= 1e-5 * np.abs(base).max()


def test_rounding_emulation():
    x = np.array([1.0, 1.0 + 2 ** -9, 1.0 + 2 ** -8, 3.14159265, -2.71828], dtype=np.float32)
    import torch
    assert np.array_equal(oracle.round_to(x, "bf16"), torch.from_numpy(x).bfloat16().float().numpy())
    assert np.array_equal(oracle.round_to(x, "f16"), torch.from_numpy(x).half().float().numpy())
    t = oracle.round_to(x, "tf32")
    assert np.all(np.abs(t - x) <= np.abs(x) * 2 ** -11)
    assert np.all((t.view(np.uint32) & 0x1FFF) == 0)
