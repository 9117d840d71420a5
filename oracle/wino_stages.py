"""Stage-by-stage CPU Winograd, numpy.  TEST INFRASTRUCTURE, not the product.

Restates the reference's numpy model of its four-kernel pipeline
(layoutTest/NCHW/data/WinoTran_NCHW.py):

    Wino_inputTran   :6-53     V[xi] = (B^T d B)[i][j],   xi = 6*i + j, 6x6 patches at stride 4
    Wino_kernelTran  :71-107   U[xi] = (G g G^T)[i][j]
    gemm             :123-145  M[xi] = V[xi]^T U[xi]      (contraction over input channels)
    Wino_OutputTran + Wino_inverseTran :147-198   Y = A^T M A, cropped to the output size

generalised to rectangular images and to F(2x2,3x3) (4x4 patches at stride 2, 16 products), which the
reference does not have; its matrices are the standard Lavin-Gray minimal-filtering form.

Buffer conventions used by every function here (the reference pads M/N/K to 128/128/8 and orders
buffers per layout; those paddings are private to its kernels and are not reproduced):

    V[xi][m][c]   m = tile index, either
                    order="ref"   : m = by*bnx*N + bx*N + n   (WinoTran_NCHW.py:52)
                    order="image" : m = n*bny*bnx + by*bnx + bx
    U[xi][k][c]
    M[xi][m][k]
    activations are logical NCHW arrays; use oracle.direct.to_layout/from_layout for NHWC/CHWN.
"""
import numpy as np


def matrices(m):
    """Return (B^T, G, A^T) for F(m x m, 3 x 3), m in {2, 4}, as float64 arrays.

    m = 4 follows the reference: B^T rows wrapedConv_NCHW.cuh:836-855 == WinoTran_NCHW.py:22-27
    (B there is this B^T transposed), G WinoTran_NCHW.py:86-91, A WinoTran_NCHW.py:181-186.
    """
    if m == 4:
        bt = np.array([[4, 0, -5, 0, 1, 0],
                       [0, -4, -4, 1, 1, 0],
                       [0, 4, -4, -1, 1, 0],
                       [0, -2, -1, 2, 1, 0],
                       [0, 2, -1, -2, 1, 0],
                       [0, 4, 0, -5, 0, 1]], dtype=np.float64)
        g = np.array([[1 / 4, 0, 0],
                      [-1 / 6, -1 / 6, -1 / 6],
                      [-1 / 6, 1 / 6, -1 / 6],
                      [1 / 24, 1 / 12, 1 / 6],
                      [1 / 24, -1 / 12, 1 / 6],
                      [0, 0, 1]], dtype=np.float64)
        at = np.array([[1, 1, 1, 1, 1, 0],
                       [0, 1, -1, 2, -2, 0],
                       [0, 1, 1, 4, 4, 0],
                       [0, 1, -1, 8, -8, 1]], dtype=np.float64)
    elif m == 2:
        bt = np.array([[1, 0, -1, 0],
                       [0, 1, 1, 0],
                       [0, -1, 1, 0],
                       [0, 1, 0, -1]], dtype=np.float64)
        g = np.array([[1, 0, 0],
                      [0.5, 0.5, 0.5],
                      [0.5, -0.5, 0.5],
                      [0, 0, 1]], dtype=np.float64)
        at = np.array([[1, 1, 1, 0],
                       [0, 1, -1, -1]], dtype=np.float64)
    else:
        raise ValueError("m must be 2 or 4")
    return bt, g, at


def tiles_per_side(size, pad, m):
    """ceil((size + 2*pad - 2) / m): `blockn` of wrapedConv_NCHW.cuh:346-350 for m = 4."""
    return -(-(size + 2 * pad - 2) // m)


def _tile_perm(n, bny, bnx, order):
    """index array p with V_order[m] = V_image[p[m]]."""
    img = np.arange(n * bny * bnx).reshape(n, bny, bnx)
    if order == "image":
        return img.reshape(-1)
    if order == "ref":
        return np.transpose(img, (1, 2, 0)).reshape(-1)
    raise ValueError(order)


def input_transform(x_nchw, pad=1, m=4, order="image", dtype=np.float64):
    """V[xi][tile][c] = (B^T d B) over the zero-padded (m+2)x(m+2) patches at stride m."""
    bt, _, _ = matrices(m)
    a = m + 2
    x = np.asarray(x_nchw, dtype=dtype)
    n, c, h, w = x.shape
    bny, bnx = tiles_per_side(h, pad, m), tiles_per_side(w, pad, m)
    hp, wp = bny * m + 2, bnx * m + 2
    xp = np.zeros((n, c, hp, wp), dtype=dtype)
    xp[:, :, pad:pad + h, pad:pad + w] = x
    s = xp.strides
    patches = np.lib.stride_tricks.as_strided(
        xp, shape=(n, c, bny, bnx, a, a), strides=(s[0], s[1], s[2] * m, s[3] * m, s[2], s[3]))
    btd = bt.astype(dtype)
    v = np.einsum("ir,ncyxrs,js->ijnyxc", btd, patches, btd, optimize=True)
    v = v.reshape(a * a, n * bny * bnx, c)
    return np.ascontiguousarray(v[:, _tile_perm(n, bny, bnx, order), :])


def filter_transform(w_kcrs, m=4, dtype=np.float64):
    """U[xi][k][c] = (G g G^T)."""
    _, g, _ = matrices(m)
    a = m + 2
    w = np.asarray(w_kcrs, dtype=dtype)
    gd = g.astype(dtype)
    u = np.einsum("ir,kcrs,js->ijkc", gd, w, gd, optimize=True)
    return np.ascontiguousarray(u.reshape(a * a, w.shape[0], w.shape[1]))


def tile_gemm(v, u, dtype=np.float64):
    """M[xi][tile][k] = sum_c V[xi][tile][c] * U[xi][k][c]  (the 16/36-way batched GEMM)."""
    return np.einsum("xtc,xkc->xtk", np.asarray(v, dtype=dtype), np.asarray(u, dtype=dtype), optimize=True)


def output_transform(mbuf, n, h, w, pad=1, m=4, order="image", bias=None, relu=False, pool=False,
                     dtype=np.float64):
    """Y (NCHW) = A^T M A per tile, cropped to (h+2p-2, w+2p-2); then + bias, ReLU, 2x2 max-pool."""
    _, _, at = matrices(m)
    a = m + 2
    mb = np.asarray(mbuf, dtype=dtype)
    k = mb.shape[2]
    bny, bnx = tiles_per_side(h, pad, m), tiles_per_side(w, pad, m)
    inv = np.argsort(_tile_perm(n, bny, bnx, order))
    mb = mb[:, inv, :].reshape(a, a, n, bny, bnx, k)
    atd = at.astype(dtype)
    y = np.einsum("pi,ijnyxk,qj->nkypxq", atd, mb, atd, optimize=True)
    y = y.reshape(n, k, bny * m, bnx * m)[:, :, :h + 2 * pad - 2, :w + 2 * pad - 2]
    if bias is not None:
        y = y + np.asarray(bias, dtype=dtype)[None, :, None, None]
    if relu:
        y = np.maximum(y, 0)
    if pool:
        oh, ow = y.shape[2] // 2, y.shape[3] // 2
        y = y[:, :, :oh * 2, :ow * 2].reshape(n, k, oh, 2, ow, 2).max(axis=(3, 5))
    return np.ascontiguousarray(y)


def round_to(x, kind):
    """Round a float array to the value grid of an MMA operand format, return float32.

    kind: "fp32" (identity), "tf32" (10-bit mantissa, round to nearest even), "bf16", "f16".
    Used to predict the error of reduced-precision variants before comparing a kernel against them.
    """
    x = np.asarray(x, dtype=np.float32)
    if kind == "fp32":
        return x
    if kind == "f16":
        return x.astype(np.float16).astype(np.float32)
    drop = {"tf32": 13, "bf16": 16}[kind]
    u = x.view(np.uint32).astype(np.uint64)
    half = np.uint64(1 << (drop - 1))
    lsb = (u >> np.uint64(drop)) & np.uint64(1)
    u = (u + half - np.uint64(1) + lsb) >> np.uint64(drop) << np.uint64(drop)
    return u.astype(np.uint32).view(np.float32).reshape(x.shape)


def winograd_conv(x_nchw, w_kcrs, pad=1, m=4, bias=None, relu=False, pool=False, storage="fp32",
                  operand="fp32"):
    """Whole chain with the rounding points of the GPU variants: activations/filters rounded to
    `storage`, transforms in float32, V and U rounded to `operand`, products accumulated wide."""
    xs = round_to(x_nchw, storage)
    ws = round_to(w_kcrs, storage)
    v = round_to(input_transform(xs, pad, m, dtype=np.float32), operand)
    u = round_to(filter_transform(ws, m, dtype=np.float64).astype(np.float32), operand)
    mb = tile_gemm(v, u, dtype=np.float64)
    n, _, h, w = x_nchw.shape
    y = output_transform(mb.astype(np.float32), n, h, w, pad, m, bias=bias, relu=relu, pool=pool,
                         dtype=np.float32)
    return round_to(y, storage)
