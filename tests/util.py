"""Shared helpers of the GPU parity tests: seeded inputs, error metrics, layout plumbing."""
import ctypes

import numpy as np

import oracle

LAYOUTS = ("NCHW", "NHWC", "CHWN")


def make_inputs(n, c, h, w, k, seed, bias=True):
    """Seeded tensors with the benchmark's distributions: x ~ U[-1,1], w ~ N(0, sqrt(2/(9c))), b ~ N(0, 0.01)."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1.0, 1.0, (n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((k, c, 3, 3)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
    b = (rng.standard_normal(k) * 0.01).astype(np.float32) if bias else None
    return x, wt, b


def maxrel(y, ref):
    """max|y - ref| / max|ref|  (element-wise relative error is undefined on the zeros ReLU produces)."""
    return float(np.abs(y.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def rel_l2(y, ref):
    d = y.astype(np.float64) - ref
    return float(np.sqrt((d * d).sum()) / max(np.sqrt((ref.astype(np.float64) ** 2).sum()), 1e-30))


def to_dev(a, torch_dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if torch_dtype is None else t.to(torch_dtype)


def run_conv(x, wt, b, layout, layout_out=None, dtype="fp32", wino=0, relu=False, pool=False, pad=1, operand=0,
             slab_images=0, out_dtype=None):
    """x, wt NCHW/KCRS numpy -> result as a float32 NCHW numpy array, through WinoConv (C ABI)."""
    import torch
    import cudnntest_b200 as cb
    lo = layout if layout_out is None else layout_out
    n, c, h, w = x.shape
    k = wt.shape[0]
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    conv = cb.WinoConv(n, c, h, w, k, layout=layout, layout_out=lo, dtype=dtype, pad=pad, wino=wino, relu=relu,
                       bias=b is not None, pool=pool, operand=operand, slab_images=slab_images, out_dtype=out_dtype)
    conv.set_filter(to_dev(oracle.filter_to_layout(wt, layout), tdt), None if b is None else to_dev(b))
    y = conv(to_dev(oracle.to_layout(x, layout), tdt))
    cb.device_status()
    return oracle.from_layout(y.float().cpu().numpy(), lo)


def desc_ptr(d):
    return ctypes.byref(d)
