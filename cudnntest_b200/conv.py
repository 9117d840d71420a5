"""Host-side objects over the C ABI: descriptors, the convolution operator, converters.

PyTorch is used for device memory and streams only; every kernel that runs is libwino's.
"""
import ctypes

import torch

from . import _lib
from ._lib import ConvDesc, LAYOUT_CODES, DTYPE_CODES, check, lib

_TORCH_DTYPE = {_lib.FP32: torch.float32, _lib.TF32: torch.float32, _lib.BF16: torch.bfloat16, _lib.FP32X3: torch.float32}


def _code(table, v):
    return table[v] if isinstance(v, str) else int(v)


def act_shape(layout, n, c, h, w):
    """Shape of an activation tensor with logical dims (n, c, h, w) stored in `layout`."""
    return {0: (n, c, h, w), 1: (n, h, w, c), 2: (c, h, w, n)}[_code(LAYOUT_CODES, layout)]


def filter_shape(layout, k, c):
    """Shape of the 3x3 filter tensor that goes with input layout `layout` (KCRS / KRSC / CRSK)."""
    return {0: (k, c, 3, 3), 1: (k, 3, 3, c), 2: (c, 3, 3, k)}[_code(LAYOUT_CODES, layout)]


_OUT_CODES = {None: _lib.OUT_SAME, "same": _lib.OUT_SAME, "fp32": _lib.OUT_FP32, "bf16": _lib.OUT_BF16}


def make_desc(n, c, h, w, k, layout="NHWC", layout_out=None, dtype="fp32", pad=1, wino=0, relu=False, bias=False,
              pool=False, operand=0, slab_images=0, out_dtype=None):
    d = ConvDesc()
    d.layout_in = _code(LAYOUT_CODES, layout)
    d.layout_out = d.layout_in if layout_out is None else _code(LAYOUT_CODES, layout_out)
    d.n, d.c, d.h, d.w, d.k, d.pad = n, c, h, w, k, pad
    d.dtype = _code(DTYPE_CODES, dtype)
    d.operand, d.wino = operand, wino
    d.relu, d.has_bias, d.pool2x2 = int(relu), int(bias), int(pool)
    d.slab_images = slab_images
    d.out_dtype = _OUT_CODES[out_dtype] if (out_dtype is None or isinstance(out_dtype, str)) else int(out_dtype)
    return d


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("libwino needs contiguous CUDA tensors")


class WinoConv:
    """One 3x3 convolution: transformed filters are computed once, the scratch is owned here.

    y = [pool2x2](relu(conv(x, w) + bias)) with x in `layout`, y in `layout_out`; out_dtype "fp32" / "bf16" stores y in
    another element type than x (the mixed-precision hand-off between layers).
    """

    def __init__(self, n, c, h, w, k, layout="NHWC", layout_out=None, dtype="fp32", pad=1, wino=0, relu=False,
                 bias=False, pool=False, operand=0, slab_images=0, device="cuda", workspace=None, out_dtype=None):
        self.desc = make_desc(n, c, h, w, k, layout, layout_out, dtype, pad, wino, relu, bias, pool, operand, slab_images,
                              out_dtype)
        L = lib()
        self.ws_bytes = L.wino_conv_workspace_bytes(ctypes.byref(self.desc))
        self.u_bytes = L.wino_filter_bytes(ctypes.byref(self.desc))
        if self.ws_bytes == 0 or self.u_bytes == 0:
            raise _lib.WinoError(_lib.E_BADARG, L.wino_last_error_string().decode())
        self.device = torch.device(device)
        self.io_dtype = _TORCH_DTYPE[self.desc.dtype]
        self.out_torch_dtype = {_lib.OUT_SAME: self.io_dtype, _lib.OUT_FP32: torch.float32,
                                _lib.OUT_BF16: torch.bfloat16}[self.desc.out_dtype]
        self.u = torch.empty(self.u_bytes, dtype=torch.uint8, device=self.device)
        if workspace is not None and workspace.numel() * workspace.element_size() >= self.ws_bytes:
            self.workspace = workspace
        else:
            self.workspace = torch.empty(self.ws_bytes, dtype=torch.uint8, device=self.device)
        oh, ow = h + 2 * pad - 2, w + 2 * pad - 2
        if pool:
            oh, ow = oh // 2, ow // 2
        self.out_shape = act_shape(self.desc.layout_out, n, k, oh, ow)
        self.bias = None

    def set_filter(self, w, bias=None):
        """w: filter tensor in the layout that goes with the input layout; bias: K floats."""
        _require_cuda(w, bias)
        if w.dtype != self.io_dtype:
            raise ValueError("filter dtype %s, expected %s" % (w.dtype, self.io_dtype))
        check(lib().wino_filter_transform(ctypes.byref(self.desc), _ptr(w), _ptr(self.u), _stream()))
        if self.desc.has_bias:
            if bias is None or bias.dtype != torch.float32 or bias.numel() != self.desc.k:
                raise ValueError("bias must be K float32 values")
            self.bias = bias
        return self

    def __call__(self, x, out=None):
        _require_cuda(x, out)
        if x.dtype != self.io_dtype:
            raise ValueError("input dtype %s, expected %s" % (x.dtype, self.io_dtype))
        if out is None:
            out = torch.empty(self.out_shape, dtype=self.out_torch_dtype, device=x.device)
        elif out.dtype != self.out_torch_dtype:
            raise ValueError("output dtype %s, expected %s" % (out.dtype, self.out_torch_dtype))
        ws = self.workspace
        check(lib().wino_conv_forward(ctypes.byref(self.desc), _ptr(x), _ptr(self.u), _ptr(self.bias), _ptr(out),
                                      _ptr(ws), ws.numel() * ws.element_size(), _stream()))
        return out


def layout_convert(x, src, dst, n, c, h, w):
    """Pure relayout of an (n, c, h, w) tensor between NCHW / NHWC / CHWN (float32 or bfloat16)."""
    _require_cuda(x)
    dt = {torch.float32: _lib.FP32, torch.bfloat16: _lib.BF16}[x.dtype]
    out = torch.empty(act_shape(dst, n, c, h, w), dtype=x.dtype, device=x.device)
    check(lib().wino_layout_convert(_code(LAYOUT_CODES, src), _code(LAYOUT_CODES, dst), n, c, h, w, dt, _ptr(x),
                                    _ptr(out), _stream()))
    return out


def maxpool2x2(x, layout, n, c, h, w):
    _require_cuda(x)
    dt = {torch.float32: _lib.FP32, torch.bfloat16: _lib.BF16}[x.dtype]
    out = torch.empty(act_shape(layout, n, c, h // 2, w // 2), dtype=x.dtype, device=x.device)
    check(lib().wino_maxpool2x2(_code(LAYOUT_CODES, layout), n, c, h, w, dt, _ptr(x), _ptr(out), _stream()))
    return out


def device_status():
    """Synchronise and raise if a device-side bounded wait gave up."""
    return check(lib().wino_device_status())
