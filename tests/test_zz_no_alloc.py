"""wino_conv_forward_static: the forward call for hosts that may not allocate device memory.

A serving process that froze its memory pool at start-up, or a plugin living under another framework's
allocator, cannot hand libwino a freshly cudaMalloc'ed scratch buffer.  This entry point keeps the slab
scratch in an array built into the library, so the test checks exactly what such a caller relies on:
the result equals wino_conv_forward's on the same tensors, a second call right after the first (reusing
the array with the previous call's contents still in it) is just as good, and a problem too large for the
array is refused with a message instead of overrunning it.

This file sorts last on purpose: a run that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest

import oracle
from util import make_inputs, maxrel, to_dev

pytestmark = pytest.mark.gpu


def _run_both(cb, n, c, h, w, k, layout, dtype, seed, wino=0, slab_images=0):
    import torch
    L = cb.lib()
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    x, wt, b = make_inputs(n, c, h, w, k, seed=seed)
    conv = cb.WinoConv(n, c, h, w, k, layout=layout, dtype=dtype, relu=True, bias=True, wino=wino, slab_images=slab_images)
    bd = to_dev(b)
    conv.set_filter(to_dev(oracle.filter_to_layout(wt, layout), tdt), bd)
    xd = to_dev(oracle.to_layout(x, layout), tdt)
    y_ref = conv(xd)
    cb.device_status()
    outs = []
    for _ in range(2):                                   # two calls in a row share the built-in scratch
        y = torch.full(conv.out_shape, float("nan"), dtype=tdt, device="cuda")
        rc = L.wino_conv_forward_static(ctypes.byref(conv.desc), xd.data_ptr(), conv.u.data_ptr(), bd.data_ptr(),
                                        y.data_ptr(), None)
        assert rc == 0, L.wino_last_error_string()
        cb.device_status()
        outs.append(y.float().cpu().numpy())
    return y_ref.float().cpu().numpy(), outs


# (layout, dtype, shape, wino, slab_images); what each case reaches inside the entry point:
CASES = [
    ("NHWC", "fp32", (5, 16, 20, 20, 24), 0, 0),       # one slab
    ("NCHW", "fp32", (3, 8, 13, 9, 40), 0, 0),         # one slab, ragged tiles
    ("NHWC", "fp32", (40, 64, 56, 56, 64), 0, 0),      # 3.6 MB of V + M per image: 16 + 16 + 8 images, the array reused by each slab
    ("CHWN", "bf16", (40, 128, 56, 56, 128), 4, 0),    # forced Winograd, 3.0 MB of V + Z per image: three slabs that start on multiples of 8
    ("CHWN", "bf16", (21, 64, 28, 28, 64), 4, 5),      # slabs of 5 images: most start off the 8-image vectors of the CHWN kernels
    ("NHWC", "bf16", (40, 64, 56, 56, 64), 0, 0),      # the direct tensor-core kernel: no scratch used at all
    ("NCHW", "bf16", (8, 64, 56, 56, 64), 0, 0),       # NHWC staging of x and y (3.2 MB each) lives in the array
    ("CHWN", "bf16", (9, 32, 14, 14, 96), 0, 0),
]


@pytest.mark.parametrize("layout,dtype,shape,wino,slab", CASES)
def test_static_scratch_matches_caller_scratch(layout, dtype, shape, wino, slab):
    import torch
    assert torch.cuda.is_available()
    import cudnntest_b200 as cb
    n, c, h, w, k = shape
    ref, outs = _run_both(cb, n, c, h, w, k, layout, dtype, seed=sum(shape), wino=wino, slab_images=slab)
    tol = 1e-4 if dtype == "fp32" else 5e-3             # the tolerances of the FP32 and BF16 parity tests
    for y in outs:
        assert np.isfinite(y).all()
        assert maxrel(y, ref.astype(np.float64)) <= tol
    assert np.array_equal(outs[0], outs[1])


def test_static_scratch_rejects_oversized_staging():
    """A BF16 NCHW layer that takes the NHWC staging route needs x and y of the whole batch in the array: 96 images
    of 64 x 56 x 56 are 38.5 MB each way, which the 64 MiB do not hold.  Refused before anything is launched."""
    import torch
    assert torch.cuda.is_available()
    import cudnntest_b200 as cb
    L = cb.lib()
    d = cb.make_desc(96, 64, 56, 56, 64, layout="NCHW", dtype="bf16")
    dummy = torch.zeros(16, device="cuda")
    rc = L.wino_conv_forward_static(ctypes.byref(d), dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(), None)
    assert rc == cb._lib.E_WORKSPACE
    msg = L.wino_last_error_string().decode()
    assert "NHWC staging" in msg and "67108864" in msg
    assert L.wino_device_status() == 0


def test_static_scratch_rejects_oversized_problem():
    import torch
    assert torch.cuda.is_available()
    import cudnntest_b200 as cb
    L = cb.lib()
    assert L.wino_static_scratch_bytes() == 64 << 20
    # one 224x224 image with 128 -> 128 channels needs ~115 MB of V + M in FP32: more than the array holds
    d = cb.make_desc(1, 128, 224, 224, 128, layout="NHWC", dtype="fp32")
    dummy = torch.zeros(16, device="cuda")
    rc = L.wino_conv_forward_static(ctypes.byref(d), dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(), None)
    assert rc == cb._lib.E_WORKSPACE
    msg = L.wino_last_error_string().decode()
    assert "built-in array holds" in msg and "67108864" in msg
    assert L.wino_device_status() == 0


def test_static_scratch_falls_back_to_slabs_when_the_staging_does_not_fit():
    """BF16 NCHW, 512 channels at 28 x 28: the engine takes the staged direct kernel at every batch, and the filter buffer
    of such a shape holds the Winograd form too.  96 images need 77 MB of NHWC staging, more than the built-in array: the
    allocation-free entry then walks the batch in Winograd slabs instead of refusing.  Different kernels, so the two
    results agree to the BF16 tolerance, not bit for bit."""
    import torch
    assert torch.cuda.is_available()
    import cudnntest_b200 as cb
    from util import rel_l2
    ref, outs = _run_both(cb, 96, 512, 28, 28, 64, "NCHW", "bf16", seed=96 + 512 + 64, wino=0, slab_images=0)
    for y in outs:
        assert np.isfinite(y).all()
        assert rel_l2(y, ref.astype(np.float64)) <= 5e-3
    assert np.array_equal(outs[0], outs[1])
