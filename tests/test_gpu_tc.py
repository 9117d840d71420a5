"""GPU parity of the tensor-core variants (tcgen05 tile GEMM): TF32 and BF16 storage with BF16/FP16 operands.

Tolerance: relative L2 error <= 5e-3 against the double-accumulating direct-convolution oracle on the
FP32 seeded tensors (the bar BASELINE.json's north_star states for TF32 and BF16).  The tile GEMM alone
is compared with a GEMM of the same rounded operands, which it must match to accumulation-order noise.
"""
import ctypes

import numpy as np
import pytest

import oracle
from util import LAYOUTS, make_inputs, maxrel, rel_l2, run_conv, to_dev

pytestmark = pytest.mark.gpu
TOL_L2 = 5e-3


@pytest.fixture(scope="module")
def cb():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    import cudnntest_b200
    cudnntest_b200.lib()
    return cudnntest_b200


@pytest.mark.parametrize("dtype,operand,kind", [("tf32", 0, "tf32"), ("bf16", 1, "bf16"), ("bf16", 2, "f16")])
@pytest.mark.parametrize("shape", [(200, 64, 64), (130, 24, 40), (1000, 256, 256), (128, 8, 200),
                                   (1000, 512, 256), (700, 512, 384), (300, 520, 512), (257, 1024, 264)])
def test_tile_gemm_alone(cb, dtype, operand, kind, shape):
    """wino_stage_gemm on random operands of the right format vs float64 GEMM of the same values.  The shapes with at
    least 256 filters and 512 channels take the CTA-pair kernel: whole and ragged pairs of row blocks (an odd number of
    blocks leaves one CTA of the last pair without rows), a half-empty and a barely started filter block, a contraction
    that is not a whole number of 128-byte slices."""
    import torch
    t, c, k = shape
    # a 1-row "image" with t tiles: n = t, h = w = 2 gives one tile per image for m = 4
    d = cb.make_desc(t, c, 2, 2, k, layout="NHWC", dtype=dtype, operand=operand, wino=4)
    L = cb.lib()
    dp = ctypes.byref(d)
    cp, kq, tp = L.wino_stage_cp(dp), L.wino_stage_kq(dp), L.wino_stage_tile_rows(dp, t)
    rng = np.random.default_rng(t + c + k)
    v = np.zeros((36, tp, cp), dtype=np.float32)
    u = np.zeros((36, k, cp), dtype=np.float32)
    v[:, :t, :c] = oracle.round_to(rng.uniform(-4, 4, (36, t, c)).astype(np.float32), kind)
    u[:, :, :c] = oracle.round_to((rng.standard_normal((36, k, c)) * 0.05).astype(np.float32), kind)
    v[:, t:, :] = np.nan      # rows past the tile count must never be read into valid outputs
    tdt = {"tf32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[kind]
    vd, ud = to_dev(v, tdt), to_dev(u, tdt)
    mm = torch.full((36, tp, kq), float("nan"), device="cuda")
    P = lambda z: ctypes.c_void_p(z.data_ptr())
    cb._lib.check(L.wino_stage_gemm(dp, P(vd), P(ud), P(mm), t, None))
    cb.device_status()
    ref = oracle.tile_gemm(v[:, :t, :c], u[:, :, :c])
    got = mm.cpu().numpy()
    assert np.isfinite(got[:, :t, :k]).all()
    assert maxrel(got[:, :t, :k], ref) <= (2e-6 if c <= 512 else 4e-6)     # FP32 accumulation noise grows with the contraction length
    assert np.all(got[:, :t, k:] == 0)


@pytest.mark.parametrize("dtype,kind,m", [("tf32", "tf32", 4), ("tf32", "tf32", 2), ("bf16", "f16", 4), ("bf16", "f16", 2)])
@pytest.mark.parametrize("shape", [(200, 64, 64), (130, 24, 40), (700, 256, 200)])
def test_rowfused_gemm_and_output_transform(cb, dtype, kind, m, shape):
    """Z = M A from the fused epilogue vs the same product computed in float64, then the remaining half of the
    output transform against the stage oracle."""
    import torch
    t, c, k = shape
    a = m + 2
    d = cb.make_desc(t, c, m, m, k, layout="NHWC", dtype=dtype, wino=m, relu=True, bias=True)   # one tile per image
    L = cb.lib()
    dp = ctypes.byref(d)
    cp, kq, tp = L.wino_stage_cp(dp), L.wino_stage_kq(dp), L.wino_stage_tile_rows(dp, t)
    rng = np.random.default_rng(t + c + k + m)
    v = np.zeros((a * a, tp, cp), dtype=np.float32)
    u = np.zeros((a * a, k, cp), dtype=np.float32)
    v[:, :t, :c] = oracle.round_to(rng.uniform(-4, 4, (a * a, t, c)).astype(np.float32), kind)
    u[:, :, :c] = oracle.round_to((rng.standard_normal((a * a, k, c)) * 0.05).astype(np.float32), kind)
    tdt = {"tf32": torch.float32, "f16": torch.float16}[kind]
    zdt = torch.float32 if dtype == "tf32" else torch.float16
    vd, ud = to_dev(v, tdt), to_dev(u, tdt)
    z = torch.full((a * m, tp, kq), float("nan"), dtype=zdt, device="cuda")
    P = lambda q: ctypes.c_void_p(q.data_ptr())
    cb._lib.check(L.wino_stage_gemm_rowfused(dp, P(vd), P(ud), P(z), t, None))
    cb.device_status()
    mm = oracle.tile_gemm(v[:, :t, :c], u[:, :, :c]).reshape(a, a, t, k)
    _, _, at = oracle.matrices(m)
    zref = np.einsum("ijtk,qj->iqtk", mm, at).reshape(a * m, t, k)
    got = z.float().cpu().numpy()
    assert np.isfinite(got[:, :t, :k]).all()
    assert maxrel(got[:, :t, :k], zref) <= (2e-6 if dtype == "tf32" else 1e-3)    # half: 2^-11 rounding of Z
    # second half of the output transform
    b = (rng.standard_normal(k) * 0.1).astype(np.float32)
    tio = torch.bfloat16 if dtype == "bf16" else torch.float32
    y = torch.full((t, m, m, k), float("nan"), dtype=tio, device="cuda")
    cb._lib.check(L.wino_stage_output_transform_rowfused(dp, P(z), P(to_dev(b)), P(y), 0, t, None))
    cb.device_status()
    yref = oracle.output_transform(mm.reshape(a * a, t, k), t, m, m, 1, m, bias=b, relu=True)   # (t, k, m, m)
    assert rel_l2(oracle.from_layout(y.float().cpu().numpy(), "NHWC"), yref) <= (1e-5 if dtype == "tf32" else 4e-3)


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("dtype,wino,operand", [("tf32", 4, 0), ("tf32", 2, 0), ("bf16", 4, 0), ("bf16", 2, 0), ("bf16", 4, 1)])
def test_conv_reduced_precision(cb, layout, dtype, wino, operand):
    n, c, h, w, k = 4, 64, 28, 28, 96
    x, wt, b = make_inputs(n, c, h, w, k, seed=31)
    y = run_conv(x, wt, b, layout, dtype=dtype, wino=wino, relu=True, operand=operand)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True)
    err = rel_l2(y, ref)
    if dtype == "bf16" and wino == 4 and operand == 1:
        # pure-BF16 operands with F(4x4,3x3) are outside the tolerance by construction; they must still
        # agree with the CPU emulation of the same rounding points
        emu = oracle.winograd_conv(x, wt, 1, 4, bias=b, relu=True, storage="bf16", operand="bf16")
        assert rel_l2(y, emu) <= 5e-3
        assert err <= 5e-2
    else:
        assert err <= TOL_L2, err


@pytest.mark.parametrize("shape", [(2, 3, 16, 16, 64), (3, 40, 9, 13, 72), (1, 512, 14, 14, 512)])
def test_conv_bf16_ragged(cb, shape):
    n, c, h, w, k = shape
    x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape))
    for layout in LAYOUTS:
        y = run_conv(x, wt, b, layout, dtype="bf16", relu=True, pool=(h % 2 == 0))
        ref = oracle.conv_f64(x, wt, bias=b, relu=True, pool=(h % 2 == 0))
        assert rel_l2(y, ref) <= TOL_L2


@pytest.mark.parametrize("dtype", ["bf16", "tf32"])
@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("shape", [(2, 3, 20, 20, 64), (1, 3, 7, 9, 40), (3, 1, 6, 6, 130), (2, 2, 5, 5, 8)])
def test_thin_input_direct_path(cb, dtype, layout, shape):
    """C <= 3 (the first VGG layer) runs the implicit-GEMM kernel; every layout, K not a multiple of 64."""
    n, c, h, w, k = shape
    x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape) + 1)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True)
    y = run_conv(x, wt, b, layout, dtype=dtype, relu=True)
    assert rel_l2(y, ref) <= TOL_L2
    for lo in LAYOUTS:
        if lo != layout:
            y2 = run_conv(x, wt, b, layout, layout_out=lo, dtype=dtype, relu=True)
            assert np.array_equal(y2, y)
    y3 = run_conv(x, wt, None, layout, dtype=dtype, pad=0)
    assert rel_l2(y3, oracle.conv_f64(x, wt, pad=0)) <= TOL_L2


@pytest.mark.parametrize("shape,pool", [((2, 64, 32, 24, 64), False), ((2, 64, 32, 24, 64), True), ((1, 128, 20, 20, 128), False),
                                        ((3, 64, 17, 13, 72), True), ((2, 128, 16, 16, 256), False), ((1, 64, 5, 37, 8), False),
                                        ((2, 128, 40, 9, 200), True), ((1, 192, 9, 9, 64), False), ((2, 256, 16, 24, 256), False),
                                        ((1, 512, 14, 14, 512), True), ((3, 256, 12, 20, 144), True), ((1, 320, 6, 6, 96), False),
                                        ((5, 64, 40, 24, 128), True), ((1, 64, 8, 16, 64), False), ((3, 64, 30, 20, 384), True),
                                        ((1, 128, 7, 9, 256), False), ((2, 64, 22, 16, 256), True), ((1, 64, 10, 8, 256), False),
                                        ((2, 64, 19, 21, 128), False), ((1, 64, 13, 10, 144), False),
                                        # 28-wide outputs: tiles of 4 whole rows over the flattened halo box (a partial last tile; pad 0)
                                        ((2, 64, 28, 28, 256), False), ((1, 128, 27, 28, 512), True), ((1, 64, 30, 30, 256), False)])
def test_direct_tensor_core_path(cb, shape, pool):
    """NHWC BF16 layers with C a multiple of 64 and no explicit tile size run the implicit-GEMM kernels (halo box +
    shifted descriptors; CTA pairs when K is a multiple of 16, the single-CTA kernel otherwise): against the oracle,
    against the Winograd path, with and without the fused pool, ragged edges, every filter-block width, resident and
    streamed filters, an odd number of tiles (a pair's spare tile is computed and dropped); K >= 256 takes the
    filters-as-M kernel with every pixel tile height (8 ... 16) and a half-empty filter block (K = 384); unpooled
    64 -> 128 / 144 layers leave through staged TMA stores that are clipped at the image and filter edges."""
    n, c, h, w, k = shape
    x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape) + 3)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True, pool=pool)
    y = run_conv(x, wt, b, "NHWC", dtype="bf16", relu=True, pool=pool)              # wino = 0 -> engine's choice: direct
    assert y.shape == ref.shape
    assert rel_l2(y, ref) <= TOL_L2
    yw = run_conv(x, wt, b, "NHWC", dtype="bf16", relu=True, pool=pool, wino=4)     # forced Winograd
    assert rel_l2(yw, ref) <= TOL_L2
    assert rel_l2(y, yw.astype(np.float64)) <= 2 * TOL_L2
    y0 = run_conv(x, wt, None, "NHWC", dtype="bf16", pad=0)
    assert rel_l2(y0, oracle.conv_f64(x, wt, pad=0)) <= TOL_L2


@pytest.mark.parametrize("shape,pool", [((2, 64, 32, 24, 64), True), ((1, 128, 20, 20, 128), False), ((3, 32, 17, 13, 80), True),
                                        ((2, 256, 16, 24, 256), True), ((1, 96, 9, 9, 64), False), ((1, 64, 12, 12, 512), False),
                                        ((1, 64, 7, 9, 256), False), ((1, 64, 14, 28, 256), True)])
@pytest.mark.parametrize("layout", ["NHWC", "NCHW", "CHWN"])
def test_direct_tensor_core_path_tf32(cb, shape, pool, layout):
    """Float storage with TF32 operands: C a multiple of 32 (up to 256) and K a multiple of 16 run the CTA-pair
    implicit-GEMM kernel with kind::tf32 (NCHW / CHWN through NHWC staging): against the oracle and the Winograd path."""
    n, c, h, w, k = shape
    x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape) + 5)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True, pool=pool)
    y = run_conv(x, wt, b, layout, dtype="tf32", relu=True, pool=pool)
    assert y.shape == ref.shape
    assert rel_l2(y, ref) <= TOL_L2
    yw = run_conv(x, wt, b, layout, dtype="tf32", relu=True, pool=pool, wino=4)
    assert rel_l2(yw, ref) <= TOL_L2


def test_second_vgg_layer_full_size(cb):
    """64 -> 64 at 224 x 224 with the fused pool, BF16 NHWC, 2 images: against the oracle."""
    x, wt, b = make_inputs(2, 64, 224, 224, 64, seed=0xC0DE0042)
    y = run_conv(x, wt, b, "NHWC", dtype="bf16", relu=True, pool=True)
    assert rel_l2(y, oracle.conv_f64(x, wt, bias=b, relu=True, pool=True)) <= TOL_L2


def test_first_vgg_layer_full_size(cb):
    """3 -> 64 at 224 x 224, BF16 NHWC, 4 images: against the oracle."""
    x, wt, b = make_inputs(4, 3, 224, 224, 64, seed=0xC0DE0041)
    y = run_conv(x, wt, b, "NHWC", dtype="bf16", relu=True)
    assert rel_l2(y, oracle.conv_f64(x, wt, bias=b, relu=True)) <= TOL_L2


def test_full_size_config1_bf16(cb):
    """BASELINE config 1 at full size, BF16 NHWC: first two images vs the oracle, slab-size invariance."""
    n, c, h, k = 64, 256, 56, 256
    x, wt, b = make_inputs(n, c, h, h, k, seed=0xC0DE0010)
    y = run_conv(x, wt, b, "NHWC", dtype="bf16", relu=True)
    y2 = run_conv(x, wt, b, "NHWC", dtype="bf16", relu=True, slab_images=7)
    assert np.array_equal(y, y2)
    ref = oracle.conv_f64(x[:2], wt, bias=b, relu=True)
    assert rel_l2(y[:2], ref) <= TOL_L2


@pytest.mark.parametrize("layout", ["NHWC", "CHWN"])
@pytest.mark.parametrize("dtype,wino", [("bf16", 2), ("bf16", 4), ("fp32", 2), ("fp32", 4)])
def test_full_size_config2(cb, layout, dtype, wino):
    """BASELINE config 2: N=64, C=K=512, 28x28, F(2x2,3x3) and F(4x4,3x3), BF16 and FP32, NHWC and CHWN.  Two images
    against the oracle; the whole batch through the property that images are independent (slab size 9 vs default)."""
    n, c, h, k = 64, 512, 28, 512
    x, wt, b = make_inputs(n, c, h, h, k, seed=0xC0DE0020)
    y = run_conv(x, wt, b, layout, dtype=dtype, wino=wino, relu=True)
    ref = oracle.conv_f64(x[:2], wt, bias=b, relu=True)
    if dtype == "fp32":
        assert maxrel(y[:2], ref) <= 1e-4
    else:
        assert rel_l2(y[:2], ref) <= TOL_L2
    y2 = run_conv(x, wt, b, layout, dtype=dtype, wino=wino, relu=True, slab_images=9)
    assert np.array_equal(y, y2)


def test_full_size_config3_bf16_nchw(cb):
    """BASELINE config 3: N=128, C=K=512, 14x14, BF16, NCHW, bias+ReLU; four images vs the oracle."""
    n, c, h, k = 128, 512, 14, 512
    x, wt, b = make_inputs(n, c, h, h, k, seed=0xC0DE0030)
    y = run_conv(x, wt, b, "NCHW", dtype="bf16", relu=True)
    ref = oracle.conv_f64(x[:4], wt, bias=b, relu=True)
    assert rel_l2(y[:4], ref) <= TOL_L2


def test_vgg16_stack_layer_by_layer_and_graph(cb):
    """The 13-layer stack (BF16 NHWC, one image): every layer's output against the oracle applied to the very
    input that layer saw on the device (so the 5e-3 bar holds per layer, with the fused pool and the activation
    ping-pong in the loop), then the same forward pass replayed from a CUDA graph gives the identical bits."""
    import torch
    from cudnntest_b200.vgg import VGG16ConvStack
    stack = VGG16ConvStack(1, layout="NHWC", dtype="bf16", seed=0xC0DE0040)
    gen = torch.Generator(device="cpu").manual_seed(7)
    x = (torch.rand(stack.in_shape, generator=gen) * 2 - 1).to(torch.bfloat16).cuda()
    cur = x
    for i, conv in enumerate(stack.convs):
        c, k, s, pool = stack.layers[i]
        out = torch.empty(conv.out_shape, dtype=torch.bfloat16, device="cuda")
        conv(cur, out=out)
        x_np = oracle.from_layout(cur.float().cpu().numpy(), "NHWC")
        w_np = stack.weights[i].to(torch.bfloat16).float().numpy()       # the filters as the device holds them
        ref = oracle.conv_f64(x_np, w_np, bias=stack.biases[i].cpu().numpy(), relu=True, pool=bool(pool))
        got = oracle.from_layout(out.float().cpu().numpy(), "NHWC")
        assert got.shape == ref.shape
        assert rel_l2(got, ref) <= TOL_L2, "layer %d (%d -> %d at %d)" % (i + 1, c, k, s)
        cur = out
    cb.device_status()
    eager = stack(x).clone()
    assert torch.equal(eager, cur)
    graph, y = stack.capture(x)
    y.zero_()
    graph.replay()
    torch.cuda.synchronize()
    cb.device_status()
    assert torch.equal(y, eager)
    assert stack.launches_per_forward >= 13


@pytest.mark.parametrize("case", [
    # n, c, h, w, k, dtype, layout_in, pool, slab_images
    (8, 512, 28, 28, 512, "bf16", "NHWC", False, 0),
    (8, 512, 28, 28, 512, "bf16", "NHWC", True, 0),
    (20, 512, 14, 14, 272, "bf16", "NHWC", False, 0),       # a ragged 256-filter block, a ragged pair of row blocks
    (40, 512, 12, 12, 256, "bf16", "NCHW", True, 32),       # two slabs, the second one less than one row block of tiles
    (12, 512, 20, 20, 512, "tf32", "NHWC", False, 0),
    (16, 512, 13, 17, 256, "tf32", "CHWN", True, 0),
])
def test_three_byte_products(cb, case):
    """Wide tensor-core layers with an NHWC result move the raw products M between the CTA-pair tile GEMM and the output
    transform as the upper 24 bits of each float (a 16-bit plane and a byte plane): the forced Winograd pipeline against
    the oracle, whole and ragged tiles, both output element types, several slabs."""
    n, c, h, w, k, dtype, layout, pool, slab = case
    x, wt, b = make_inputs(n, c, h, w, k, seed=n + h + k)
    y = run_conv(x, wt, b, layout, layout_out="NHWC", dtype=dtype, relu=True, pool=pool, wino=4, slab_images=slab)
    ref = oracle.conv_f64(x, wt, b, pad=1, relu=True, pool=pool)
    assert y.shape == ref.shape
    assert rel_l2(y, ref) <= TOL_L2
