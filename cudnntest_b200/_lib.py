"""ctypes binding of libwino.so (the C ABI declared in include/wino.h).

The library is built in-tree by ``build()`` (nvcc, sm_100a only) and loaded from
``cudnntest_b200/libwino.so``.  There is no fallback: if the shared object is missing or a symbol
declared in the header is absent, loading raises.
"""
import ctypes
import os
import re
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libwino.so")
_HEADER = os.path.join(os.path.dirname(_HERE), "include", "wino.h")

NCHW, NHWC, CHWN = 0, 1, 2
FP32, TF32, BF16, FP32X3 = 0, 1, 2, 3
OPERAND_AUTO, OPERAND_BF16, OPERAND_F16 = 0, 1, 2
OUT_SAME, OUT_FP32, OUT_BF16 = 0, 1, 2
OK, E_BADARG, E_UNSUPPORTED, E_WORKSPACE, E_CUDA, E_TIMEOUT = 0, -1, -2, -3, -4, -5
LAYOUT_CODES = {"NCHW": NCHW, "NHWC": NHWC, "CHWN": CHWN}
DTYPE_CODES = {"fp32": FP32, "tf32": TF32, "bf16": BF16, "fp32x3": FP32X3}


class WinoError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("libwino error %d: %s" % (code, message))
        self.code = code


class ConvDesc(ctypes.Structure):
    """struct wino_conv_desc"""
    _fields_ = [(n, ctypes.c_int) for n in (
        "layout_in", "layout_out", "n", "c", "h", "w", "k", "pad", "dtype", "operand", "wino",
        "relu", "has_bias", "pool2x2", "slab_images", "out_dtype")]


def declared_symbols():
    """Names of every function declared in include/wino.h."""
    text = open(_HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wino_[a-z0-9_]+)\s*\(", text)))


def build(force=False, verbose=False):
    """Compile every CUDA translation unit for sm_100a and link cudnntest_b200/libwino.so."""
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), "-j8"]
    if force:
        cmd.append("-B")
    subprocess.check_call(cmd, stdout=None if verbose else subprocess.DEVNULL)
    # the harness executables (layoutCompare, layoutTest, netTest) link libwino and, for the comparator, cuDNN
    hcmd = ["make", "-C", os.path.join(_HERE, "harness"), "-j3"] + (["-B"] if force else [])
    subprocess.check_call(hcmd, stdout=None if verbose else subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_SO):
        raise ImportError("libwino.so is not built: run `python -c 'import __graft_entry__ as g; g.build()'` "
                          "or `make -C cudnntest_b200/csrc` (there is no CPU or PyTorch fallback)")
    L = ctypes.CDLL(_SO)
    missing = [s for s in declared_symbols() if not hasattr(L, s)]
    if missing:
        raise ImportError("libwino.so lacks symbols declared in wino.h: %s" % missing)
    P, I, V, SZ = ctypes.POINTER(ConvDesc), ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
    L.wino_last_error_string.restype = ctypes.c_char_p
    L.wino_last_error_string.argtypes = []
    L.wino_version.restype = I
    L.wino_device_status.restype = I
    L.wino_filter_bytes.restype = SZ
    L.wino_filter_bytes.argtypes = [P]
    L.wino_conv_workspace_bytes.restype = SZ
    L.wino_conv_workspace_bytes.argtypes = [P]
    L.wino_filter_transform.argtypes = [P, V, V, V]
    L.wino_conv_forward.argtypes = [P, V, V, V, V, V, SZ, V]
    L.wino_static_scratch_bytes.restype = SZ
    L.wino_static_scratch_bytes.argtypes = []
    L.wino_conv_forward_static.argtypes = [P, V, V, V, V, V]
    L.wino_conv_forward_static.restype = I
    L.wino_wraped_conv.argtypes = [I, I, I, I, ctypes.POINTER(I), I, I, V, V, V, V, V, ctypes.POINTER(V)]
    L.wino_layout_convert.argtypes = [I, I, I, I, I, I, I, V, V, V]
    L.wino_maxpool2x2.argtypes = [I, I, I, I, I, I, V, V, V]
    L.wino_selftest_wait_timeout.argtypes = [I, V]
    L.wino_selftest_wait_timeout.restype = I
    L.wino_stage_tile_rows.restype = ctypes.c_longlong
    L.wino_stage_tile_rows.argtypes = [P, I]
    L.wino_stage_cp.argtypes = [P]
    L.wino_stage_kq.argtypes = [P]
    L.wino_stage_input_transform.argtypes = [P, V, I, I, V, V]
    L.wino_stage_gemm.argtypes = [P, V, V, V, I, V]
    L.wino_stage_output_transform.argtypes = [P, V, V, V, I, I, V]
    L.wino_stage_gemm_rowfused.argtypes = [P, V, V, V, I, V]
    L.wino_stage_output_transform_rowfused.argtypes = [P, V, V, V, I, I, V]
    for name in ("wino_filter_transform", "wino_conv_forward", "wino_wraped_conv", "wino_layout_convert",
                 "wino_maxpool2x2", "wino_stage_cp", "wino_stage_kq", "wino_stage_input_transform",
                 "wino_stage_gemm", "wino_stage_output_transform", "wino_stage_gemm_rowfused",
                 "wino_stage_output_transform_rowfused"):
        getattr(L, name).restype = I
    _lib = L
    return L


def check(code):
    if code != OK:
        raise WinoError(code, lib().wino_last_error_string().decode())
    return code
