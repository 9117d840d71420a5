"""cudnntest_b200 — B200-native Winograd 3x3 convolution behind the entry points of Elon-Wang/cudnnTest.

The product is ``libwino.so`` (hand-written sm_100a CUDA behind the C ABI of ``include/wino.h``); this
package is its Python host side: the ctypes binding, the operator objects and the mirror of the
reference's ``wrapedConv_*`` / ``layoutManager`` / ``convLayoutTrans_*`` interface.
"""
from ._lib import (build, lib, WinoError, ConvDesc, declared_symbols, NCHW, NHWC, CHWN, FP32, TF32, BF16, FP32X3,  # noqa: F401
                   OPERAND_AUTO, OPERAND_BF16, OPERAND_F16, OUT_SAME, OUT_FP32, OUT_BF16)
from .conv import WinoConv, make_desc, layout_convert, maxpool2x2, device_status, act_shape, filter_shape  # noqa: F401
from .wraped import (DataLayout, layoutManager, legacy_workspace_floats, wrapedConv_NCHW, wrapedConv_NHWC,  # noqa: F401
                     wrapedConv_CHWN, convLayoutTrans_CHWN_to_NCHW, convLayoutTrans_CHWN_to_NHWC,
                     convLayoutTrans_NHWC_to_NCHW, convLayoutTrans_NHWC_to_CHWN, convLayoutTrans_NCHW_to_NHWC,
                     convLayoutTrans_NCHW_to_CHWN)
