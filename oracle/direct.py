"""ctypes front-end of ``wino_ref.cpp`` (the C++ restatement of the reference's ``Conv_*``).

Test infrastructure only.  Layout codes follow the reference's ``enum class DataLayout``
(comparison/DataLayoutTrans.cuh:587-591): 0 NCHW, 1 NHWC, 2 CHWN; the filter layout follows the input
layout (KCRS / KRSC / CRSK).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libwino_ref.so")
LAYOUTS = {"NCHW": 0, "NHWC": 1, "CHWN": 2}
_lib = None


def build(force=False):
    """Compile ``wino_ref.cpp`` into ``oracle/libwino_ref.so`` (g++, OpenMP)."""
    src = os.path.join(_HERE, "wino_ref.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-B", "-C", _HERE, "libwino_ref.so"], stdout=subprocess.DEVNULL)
    return _SO


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        fp = ctypes.POINTER(ctypes.c_float)
        sig = [ctypes.c_int] * 8 + [fp, fp, fp, ctypes.c_int, ctypes.c_int, fp]
        for name in ("ref_conv_f64", "ref_conv_f32", "ref_conv_f32_plain"):
            getattr(_lib, name).argtypes = sig
            getattr(_lib, name).restype = None
        _lib.ref_maxpool2x2.argtypes = [ctypes.c_int] * 5 + [fp, fp]
        _lib.ref_maxpool2x2.restype = None
        _lib.ref_num_threads.restype = ctypes.c_int
    return _lib


def _code(layout):
    return LAYOUTS[layout] if isinstance(layout, str) else int(layout)


def _dims(x, layout):
    """Logical (N, C, H, W) of an activation array stored in `layout`."""
    s = x.shape
    return {0: (s[0], s[1], s[2], s[3]), 1: (s[0], s[3], s[1], s[2]), 2: (s[3], s[0], s[1], s[2])}[_code(layout)]


def _shape(layout, n, c, h, w):
    return {0: (n, c, h, w), 1: (n, h, w, c), 2: (c, h, w, n)}[_code(layout)]


def to_layout(x_nchw, layout):
    """NCHW array -> contiguous array in `layout`."""
    perm = {0: (0, 1, 2, 3), 1: (0, 2, 3, 1), 2: (1, 2, 3, 0)}[_code(layout)]
    return np.ascontiguousarray(np.transpose(x_nchw, perm))


def from_layout(x, layout):
    """array in `layout` -> contiguous NCHW array."""
    perm = {0: (0, 1, 2, 3), 1: (0, 3, 1, 2), 2: (3, 0, 1, 2)}[_code(layout)]
    return np.ascontiguousarray(np.transpose(x, perm))


def filter_to_layout(w_kcrs, layout):
    """KCRS filters -> the filter layout that goes with activation `layout` (KCRS / KRSC / CRSK)."""
    perm = {0: (0, 1, 2, 3), 1: (0, 2, 3, 1), 2: (1, 2, 3, 0)}[_code(layout)]
    return np.ascontiguousarray(np.transpose(w_kcrs, perm))


def _filter_k(w, layout):
    return {0: w.shape[0], 1: w.shape[0], 2: w.shape[3]}[_code(layout)]


def _run(fn, x, w, bias, pad, relu, pool, layout_in, layout_out):
    lib = _load()
    li, lo = _code(layout_in), _code(layout_out if layout_out is not None else layout_in)
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, c, h, wd = _dims(x, li)
    k = _filter_k(w, li)
    oh, ow = h + 2 * pad - 2, wd + 2 * pad - 2
    if pool:
        oh, ow = oh // 2, ow // 2
    y = np.empty(_shape(lo, n, k, oh, ow), dtype=np.float32)
    fp = ctypes.POINTER(ctypes.c_float)
    b = None
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        b = bias.ctypes.data_as(fp)
    getattr(lib, fn)(li, lo, n, c, h, wd, k, pad, x.ctypes.data_as(fp), w.ctypes.data_as(fp), b,
                     int(bool(relu)), int(bool(pool)), y.ctypes.data_as(fp))
    return y


def conv_f64(x, w, bias=None, pad=1, relu=False, pool=False, layout="NCHW", layout_out=None):
    """The oracle: direct 3x3 cross-correlation, double accumulation (Conv_* restated)."""
    return _run("ref_conv_f64", x, w, bias, pad, relu, pool, layout, layout_out)


def conv_f32_plain(x, w, bias=None, pad=1, relu=False, pool=False, layout="NCHW", layout_out=None):
    """Same loop nest with float accumulation (the reference's float32 arithmetic)."""
    return _run("ref_conv_f32_plain", x, w, bias, pad, relu, pool, layout, layout_out)


def conv_f32(x, w, bias=None, pad=1, relu=False, pool=False, layout="NCHW", layout_out=None):
    """The timed CPU baseline: float accumulation, all host threads, SIMD over output channels."""
    return _run("ref_conv_f32", x, w, bias, pad, relu, pool, layout, layout_out)


def maxpool2x2(x, layout="NCHW"):
    lib = _load()
    li = _code(layout)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, c, h, w = _dims(x, li)
    y = np.empty(_shape(li, n, c, h // 2, w // 2), dtype=np.float32)
    fp = ctypes.POINTER(ctypes.c_float)
    lib.ref_maxpool2x2(li, n, c, h, w, x.ctypes.data_as(fp), y.ctypes.data_as(fp))
    return y


def num_threads():
    return int(_load().ref_num_threads())


def set_num_threads(n):
    """Threads of the float32 baseline (conv_f32); the environment's OMP_NUM_THREADS is only the default."""
    _load().ref_set_num_threads(int(n))
