"""CPU-side checks of the C ABI: the library loads, exports what include/wino.h declares, validates
descriptors and sizes buffers — no compute call needs a GPU here."""
import ctypes
import math

import pytest

import cudnntest_b200 as cb


@pytest.fixture(scope="module")
def L():
    return cb.lib()


def test_exports_every_declared_symbol(L):
    names = cb.declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), n
    assert L.wino_version() >= 100


def test_descriptor_validation(L):
    good = cb.make_desc(8, 64, 56, 56, 64, layout="NCHW")
    assert L.wino_conv_workspace_bytes(ctypes.byref(good)) > 0
    for field, value in (("pad", 2), ("wino", 3), ("dtype", 7), ("layout_in", 5), ("c", 0), ("k", -1), ("operand", 9)):
        d = cb.make_desc(8, 64, 56, 56, 64, layout="NCHW", dtype="bf16")
        setattr(d, field, value)
        assert L.wino_conv_workspace_bytes(ctypes.byref(d)) == 0, field
        assert L.wino_last_error_string()
    assert L.wino_conv_workspace_bytes(None) == 0


@pytest.mark.parametrize("shape", [(8, 64, 56, 56, 64), (1, 20, 13, 10, 12), (128, 512, 14, 14, 512)])
@pytest.mark.parametrize("m", [2, 4])
def test_buffer_sizes_split_operands(L, shape, m):
    """FP32X3: the transformed filters keep a TF32 head and a TF32 tail (rows of 2 * Cp floats); V and M are plain
    float buffers of the FP32 variant's size (V is split inside the tile GEMM)."""
    n, c, h, w, k = shape
    d = cb.make_desc(n, c, h, w, k, dtype="fp32x3", wino=m)
    d32 = cb.make_desc(n, c, h, w, k, dtype="fp32", wino=m)
    dp, dp32 = ctypes.byref(d), ctypes.byref(d32)
    a, cp, kq = m + 2, math.ceil(c / 8) * 8, math.ceil(k / 8) * 8
    assert L.wino_stage_cp(dp) == cp and L.wino_stage_kq(dp) == kq
    assert L.wino_filter_bytes(dp) == 2 * L.wino_filter_bytes(dp32) == a * a * k * 2 * cp * 4
    d.slab_images = d32.slab_images = n
    assert L.wino_conv_workspace_bytes(dp) == L.wino_conv_workspace_bytes(dp32)


@pytest.mark.parametrize("shape", [(8, 64, 56, 56, 64), (64, 256, 56, 56, 256), (1, 3, 224, 224, 64), (128, 512, 14, 14, 512)])
@pytest.mark.parametrize("dtype", ["fp32", "tf32", "bf16"])
@pytest.mark.parametrize("m", [2, 4])
def test_buffer_sizes(L, shape, dtype, m):
    n, c, h, w, k = shape
    d = cb.make_desc(n, c, h, w, k, dtype=dtype, wino=m)
    dp = ctypes.byref(d)
    a = m + 2
    cp, kq = L.wino_stage_cp(dp), L.wino_stage_kq(dp)
    assert cp == math.ceil(c / 8) * 8 and kq == math.ceil(k / 8) * 8
    es = 2 if dtype == "bf16" else 4
    assert L.wino_filter_bytes(dp) == a * a * k * cp * es
    tiles = math.ceil(h / m) * math.ceil(w / m)
    assert L.wino_stage_tile_rows(dp, 3) == math.ceil(3 * tiles / 128) * 128
    # scratch = V + product buffer of one slab; the product buffer is M (a*a float planes) for FP32 and for wide
    # layers, Z (a*m planes, half for BF16) where the row-fused tile GEMM is used
    ws = L.wino_conv_workspace_bytes(dp)
    v_img = a * a * tiles * cp * es
    assert ws >= v_img + a * m * tiles * kq * 2
    d.slab_images = n
    ws_all = L.wino_conv_workspace_bytes(dp)
    assert ws_all >= n * (v_img + a * m * tiles * kq * 2)
    if dtype == "fp32":
        assert ws_all >= n * (v_img + a * a * tiles * kq * 4)
    assert ws_all <= n * (v_img + a * a * tiles * kq * 4) + a * a * 128 * (cp * es + kq * 4) + 4096


@pytest.mark.parametrize("layout", ["NCHW", "NHWC", "CHWN"])
@pytest.mark.parametrize("dtype", ["fp32", "tf32", "bf16", "fp32x3"])
@pytest.mark.parametrize("chw", [(3, 224, 224, 64), (64, 56, 56, 64), (256, 56, 56, 256), (512, 28, 28, 512), (512, 14, 14, 512)])
def test_filter_buffer_does_not_depend_on_the_batch(L, layout, dtype, chw):
    """Weights are transformed once and used with any batch size: the size (and with it the format) of the filter
    buffer must not change with n, although the engine's kernel choice does (512 channels at 28 x 28: direct kernel
    for fewer than 4 images, Winograd from there on, so that buffer holds both forms)."""
    c, h, w, k = chw
    sizes = {L.wino_filter_bytes(ctypes.byref(cb.make_desc(n, c, h, w, k, layout=layout, dtype=dtype))) for n in (1, 8, 127, 128, 256)}
    assert len(sizes) == 1 and 0 not in sizes
    if dtype == "bf16" and c == 512 and h == 28:
        u_wino = 36 * k * c * 2
        assert sizes == {u_wino + 9 * k * c * 2}


def test_legacy_workspaces_cover_the_slabs(L):
    """The reference callers' minimum buffer sizes hold this library's V, U, M for any slab."""
    for (n, h, c, k) in ((1, 224, 3, 64), (8, 56, 64, 64), (64, 28, 512, 512), (3, 14, 20, 130)):
        vf, uf, mf = cb.legacy_workspace_floats(n, h, c, k, 1)
        d = cb.make_desc(n, c, h, h, k, dtype="fp32", wino=4)
        dp = ctypes.byref(d)
        cp, kq, tp = L.wino_stage_cp(dp), L.wino_stage_kq(dp), L.wino_stage_tile_rows(dp, n)
        assert 36 * tp * cp <= vf and 36 * k * cp <= uf and 36 * tp * kq <= mf


def test_no_cpu_fallback(L):
    """Without a CUDA device every compute entry point fails loudly with WINO_E_CUDA."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    d = cb.make_desc(1, 8, 8, 8, 8)
    buf = (ctypes.c_float * 16)()
    rc = L.wino_filter_transform(ctypes.byref(d), buf, buf, None)
    assert rc == cb._lib.E_CUDA
    assert b"no CPU path" in L.wino_last_error_string()
    assert L.wino_device_status() == cb._lib.E_CUDA
