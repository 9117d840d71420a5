"""GPU parity at the sizes and routings the benchmark actually runs.

* BASELINE config 1 (N=64, C=K=256, 56 x 56, bias + ReLU) at full size in all nine {FP32, TF32, BF16} x {NCHW, NHWC,
  CHWN} variants: at this size the engine picks other kernel templates than the small parity cases do (CTA-pair direct
  kernels with filters as the MMA's M dimension, the NHWC staging route of the other layouts).
* The VGG-16 stack at batch 256, BF16 NHWC, i.e. the routing bench.py times (the 512 -> 512 layers at 28 x 28 go
  through the Winograd pipeline there, not through the direct kernel that a batch of 1 selects).
* Convolutions that change layout (comparison/DataLayoutTrans.cuh:9, 101, 192, 309, 418, 502) in the tensor-core
  variants, through the direct kernel, its staging route and the Winograd route.
* Filters transformed once and used with batches on both sides of the engine's batch-size switch.
* The mixed-precision hand-off: a BF16 layer that writes FP32 (in another layout), and the reverse.

Tolerances: FP32 max|d|/max|ref| <= 1e-4; TF32 / BF16 relative L2 <= 5e-3, against the double-accumulating oracle.
"""
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


@pytest.fixture(scope="module")
def config1():
    n, c, h, k = 64, 256, 56, 256
    x, wt, b = make_inputs(n, c, h, h, k, seed=0xC0DE0010)
    ref = oracle.conv_f64(x[:2], wt, bias=b, relu=True)
    return x, wt, b, ref


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("dtype", ["fp32", "tf32", "bf16"])
def test_full_size_config1(cb, config1, dtype, layout):
    """Two images against the oracle; the whole batch through the independence of images: a run with slabs of 7
    images (Winograd route) or on the last 23 images alone (any route) gives the same bits."""
    x, wt, b, ref = config1
    y = run_conv(x, wt, b, layout, dtype=dtype, relu=True)
    assert np.isfinite(y).all()
    if dtype == "fp32":
        assert maxrel(y[:2], ref) <= 1e-4
        y2 = run_conv(x, wt, b, layout, dtype=dtype, relu=True, slab_images=7)
        assert np.array_equal(y, y2)
    else:
        assert rel_l2(y[:2], ref) <= TOL_L2
    tail = run_conv(x[-23:], wt, b, layout, dtype=dtype, relu=True)
    assert np.array_equal(tail, y[-23:])


def test_vgg16_stack_batch256_routing(cb):
    """The benchmark's own configuration: 13 layers, batch 256, BF16 NHWC.  Images 0 and 255 of every layer's output
    against the oracle applied to what that layer read on the device."""
    import torch
    from cudnntest_b200.vgg import VGG16ConvStack
    batch = 256
    stack = VGG16ConvStack(batch, layout="NHWC", dtype="bf16", seed=0xC0DE0040)
    gen = torch.Generator(device="cpu").manual_seed(11)
    x = (torch.rand(stack.in_shape, generator=gen) * 2 - 1).to(torch.bfloat16).cuda()
    pick = torch.tensor([0, batch - 1], device="cuda")
    cur = x
    for i, conv in enumerate(stack.convs):
        c, k, s, pool = stack.layers[i]
        out = stack.act[i % 2][: int(np.prod(conv.out_shape))].view(conv.out_shape)
        x_np = oracle.from_layout(cur.index_select(0, pick).float().cpu().numpy(), "NHWC")
        conv(cur, out=out)
        w_np = stack.weights[i].to(torch.bfloat16).float().numpy()
        ref = oracle.conv_f64(x_np, w_np, bias=stack.biases[i].cpu().numpy(), relu=True, pool=bool(pool))
        got = oracle.from_layout(out.index_select(0, pick).float().cpu().numpy(), "NHWC")
        assert got.shape == ref.shape
        assert rel_l2(got, ref) <= TOL_L2, "layer %d (%d -> %d at %d)" % (i + 1, c, k, s)
        cur = out
    cb.device_status()
    final = cur.clone()
    graph, y = stack.capture(x)
    y.zero_()
    graph.replay()
    torch.cuda.synchronize()
    cb.device_status()
    assert torch.equal(y, final)


@pytest.mark.parametrize("dtype", ["bf16", "tf32"])
@pytest.mark.parametrize("shape,pool", [((3, 64, 18, 14, 96), False), ((3, 64, 18, 14, 96), True),      # direct kernel + staging
                                        ((2, 64, 18, 14, 256), False), ((2, 64, 18, 14, 256), True),    # filters-as-M kernel: NCHW stored in place, odd row pitches
                                        ((1, 64, 12, 28, 256), False), ((1, 64, 6, 40, 384), True),     # ... 8-byte and 16-byte vectors, clipped tiles
                                        ((1, 64, 14, 28, 256), True),                                   # ... flattened-row tiles with the pool
                                        ((2, 328, 14, 10, 72), False), ((2, 328, 14, 10, 72), True)])   # Winograd route
def test_cross_layout_tensor_core(cb, dtype, shape, pool):
    """All nine (source, destination) pairs: each result against the oracle, and the same numbers whatever the
    destination layout is."""
    n, c, h, w, k = shape
    x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape) + 9)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True, pool=pool)
    for src in LAYOUTS:
        same = run_conv(x, wt, b, src, dtype=dtype, relu=True, pool=pool)
        assert rel_l2(same, ref) <= TOL_L2, (src,)
        for dst in LAYOUTS:
            if dst == src:
                continue
            y = run_conv(x, wt, b, src, layout_out=dst, dtype=dtype, relu=True, pool=pool)
            assert y.shape == ref.shape
            assert rel_l2(y, ref) <= TOL_L2, (src, dst)
            assert rel_l2(y, same.astype(np.float64)) <= TOL_L2


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_filters_transformed_once_serve_every_batch_size(cb, layout):
    """512 -> 512 at 28 x 28, BF16: in NHWC the engine runs the direct kernel for fewer than 4 images and the Winograd
    pipeline from there on (in NCHW the staged direct kernel at every batch).  One filter buffer, written through a descriptor of either batch size, serves both."""
    import torch
    c, h, k = 512, 28, 512
    x, wt, b = make_inputs(130, c, h, h, k, seed=0xC0DE0021)
    ref = oracle.conv_f64(x[:2], wt, bias=b, relu=True)
    wd = to_dev(oracle.filter_to_layout(wt, layout), torch.bfloat16)
    bd = to_dev(b)
    big = cb.WinoConv(130, c, h, h, k, layout=layout, dtype="bf16", relu=True, bias=True)
    small = cb.WinoConv(2, c, h, h, k, layout=layout, dtype="bf16", relu=True, bias=True)
    assert big.u_bytes == small.u_bytes
    xb = to_dev(oracle.to_layout(x, layout), torch.bfloat16)
    xs = to_dev(oracle.to_layout(x[:2], layout), torch.bfloat16)
    for owner, other in ((big, small), (small, big)):
        owner.set_filter(wd, bd)
        other.u, other.bias = owner.u, bd               # the other batch size reads the same buffer
        yb = oracle.from_layout(big(xb).float().cpu().numpy(), layout)
        ys = oracle.from_layout(small(xs).float().cpu().numpy(), layout)
        cb.device_status()
        assert rel_l2(yb[:2], ref) <= TOL_L2
        assert rel_l2(ys, ref) <= TOL_L2
        owner.u = torch.zeros_like(owner.u)             # a fresh buffer for the other direction


@pytest.mark.parametrize("src,dst", [("CHWN", "NCHW"), ("NHWC", "NHWC"), ("NCHW", "CHWN")])
@pytest.mark.parametrize("shape,pool", [((3, 64, 14, 14, 64), True), ((2, 3, 12, 12, 40), False), ((2, 200, 9, 11, 72), False)])
def test_mixed_precision_hand_off(cb, src, dst, shape, pool):
    """A BF16 layer that stores FP32 (what the last convolution of the reference's network does for its FP32
    classifier, together with the CHWN -> NCHW change of netTest/cudnn_test_0124/VGG_Batched/vggCUDNN.cu:173-176),
    and a TF32 layer that stores BF16."""
    import torch
    n, c, h, w, k = shape
    x, wt, b = make_inputs(n, c, h, w, k, seed=sum(shape) + 13)
    ref = oracle.conv_f64(x, wt, bias=b, relu=True, pool=pool)
    for dtype, out_dtype, tout in (("bf16", "fp32", torch.float32), ("tf32", "bf16", torch.bfloat16)):
        tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
        conv = cb.WinoConv(n, c, h, w, k, layout=src, layout_out=dst, dtype=dtype, relu=True, bias=True, pool=pool,
                           out_dtype=out_dtype)
        conv.set_filter(to_dev(oracle.filter_to_layout(wt, src), tdt), to_dev(b))
        y = conv(to_dev(oracle.to_layout(x, src), tdt))
        cb.device_status()
        assert y.dtype == tout
        got = oracle.from_layout(y.float().cpu().numpy(), dst)
        assert rel_l2(got, ref) <= TOL_L2, (dtype, out_dtype)
        if out_dtype == "fp32":
            # the FP32 result is the BF16 layer's result before its final rounding: rounding it gives the same layer
            same = run_conv(x, wt, b, src, layout_out=dst, dtype=dtype, relu=True, pool=pool, wino=4)
            assert np.array_equal(got.astype(np.float32), got)      # stored as float
            assert rel_l2(oracle.round_to(got, "bf16"), same.astype(np.float64)) <= 1e-6
