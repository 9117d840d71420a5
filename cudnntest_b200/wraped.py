"""Python mirror of the reference's operator interface, over the C ABI.

Same names, argument order and behaviour as the reference's host functions
(comparison/wrapedConv_NCHW.cuh:8, wrapedConv_NHWC.cuh:8, wrapedConv_CHWN.cuh:8,
comparison/DataLayoutTrans.cuh:9-651): FP32, F(4x4,3x3), square images, caller-owned workspaces with
the reference's minimum sizes, synchronous.  `chn` is in/out in the reference (``int&``); here the new
channel count is returned.
"""
import ctypes
import enum

from ._lib import check, lib


class DataLayout(enum.IntEnum):
    """enum class DataLayout, comparison/DataLayoutTrans.cuh:587-591"""
    NCHW = 0
    NHWC = 1
    CHWN = 2


def legacy_workspace_floats(bat4Conv, inside, chn, numOfFilter, padding=1):
    """Minimum sizes (floats) of inputTran_gpu, filterTran_gpu, gemmOutput_gpu the reference callers
    allocate (layoutTest/NCHW/convModule_NCHW_padding.cu:44-50)."""
    bn = -(-(inside + 2 * padding - 2) // 4)
    mp = -(-(bat4Conv * bn * bn) // 128) * 128
    np_ = -(-numOfFilter // 128) * 128
    kp = -(-chn // 8) * 8
    return 36 * mp * kp, 36 * np_ * kp, 36 * mp * np_


def layoutManager(srcLayout, dstLayout, bat4Conv, inside, chn, numOfFilter, padding, input, weights, inputTran_gpu,
                  filterTran_gpu, gemmOutput_gpu, output):
    """layoutManager, comparison/DataLayoutTrans.cuh:594-651.  Returns the new channel count."""
    c = ctypes.c_int(chn)
    out_ptr = ctypes.c_void_p(output.data_ptr())
    check(lib().wino_wraped_conv(int(srcLayout), int(dstLayout), bat4Conv, inside, ctypes.byref(c), numOfFilter, padding,
                                 ctypes.c_void_p(input.data_ptr()), ctypes.c_void_p(weights.data_ptr()),
                                 ctypes.c_void_p(inputTran_gpu.data_ptr()), ctypes.c_void_p(filterTran_gpu.data_ptr()),
                                 ctypes.c_void_p(gemmOutput_gpu.data_ptr()), ctypes.byref(out_ptr)))
    return c.value


def _same(layout):
    def f(bat4Conv, inside, chn, numOfFilter, padding, m1, m2, inputTran_gpu, filterTran_gpu, gemmOutput_gpu, output):
        return layoutManager(layout, layout, bat4Conv, inside, chn, numOfFilter, padding, m1, m2, inputTran_gpu,
                             filterTran_gpu, gemmOutput_gpu, output)
    f.__name__ = "wrapedConv_" + layout.name
    f.__doc__ = "wrapedConv_%s, comparison/wrapedConv_%s.cuh:8" % (layout.name, layout.name)
    return f


def _cross(src, dst):
    def f(bat4Conv, inside, chn, numOfFilter, padding, m1, m2, inputTran_gpu, filterTran_gpu, gemmOutput_gpu, output):
        return layoutManager(src, dst, bat4Conv, inside, chn, numOfFilter, padding, m1, m2, inputTran_gpu,
                             filterTran_gpu, gemmOutput_gpu, output)
    f.__name__ = "convLayoutTrans_%s_to_%s" % (src.name, dst.name)
    f.__doc__ = "convLayoutTrans_%s_to_%s, comparison/DataLayoutTrans.cuh:9-584" % (src.name, dst.name)
    return f


wrapedConv_NCHW = _same(DataLayout.NCHW)
wrapedConv_NHWC = _same(DataLayout.NHWC)
wrapedConv_CHWN = _same(DataLayout.CHWN)
convLayoutTrans_CHWN_to_NCHW = _cross(DataLayout.CHWN, DataLayout.NCHW)
convLayoutTrans_CHWN_to_NHWC = _cross(DataLayout.CHWN, DataLayout.NHWC)
convLayoutTrans_NHWC_to_NCHW = _cross(DataLayout.NHWC, DataLayout.NCHW)
convLayoutTrans_NHWC_to_CHWN = _cross(DataLayout.NHWC, DataLayout.CHWN)
convLayoutTrans_NCHW_to_NHWC = _cross(DataLayout.NCHW, DataLayout.NHWC)
convLayoutTrans_NCHW_to_CHWN = _cross(DataLayout.NCHW, DataLayout.CHWN)
