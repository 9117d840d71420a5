"""VGG-16 convolution stack on the Winograd engine: 13 3x3 pad-1 convolutions, bias + ReLU after each,
2x2 max-pool after each block — the conv part of the reference's network path
(netTest/cudnn_test_0124/VGG_Batched/Network.h:603-669, layer table vggCUDNN.cu:154-180).

Where the reference runs conv, bias, ReLU and pool as four to seven kernels per layer, each layer here
is one ``wino_conv_forward`` call whose output transform applies bias, ReLU and (at block ends) the
pool.  Weights are random He-initialised (the pretrained ``vggData/conv*.bin`` are not shipped with the
reference); activations ping-pong between two buffers and all layers share one scratch buffer.
"""
import ctypes
import math

import torch

from . import _lib
from .conv import WinoConv, act_shape, make_desc

# (input channels, filters, input side, pool after)
VGG16_CONV = [
    (3, 64, 224, False), (64, 64, 224, True),
    (64, 128, 112, False), (128, 128, 112, True),
    (128, 256, 56, False), (256, 256, 56, False), (256, 256, 56, True),
    (256, 512, 28, False), (512, 512, 28, False), (512, 512, 28, True),
    (512, 512, 14, False), (512, 512, 14, False), (512, 512, 14, True),
]


def direct_flops_per_image(layers=VGG16_CONV):
    """Direct-convolution-equivalent FLOPs of the stack for one image: sum of 2*K*C*H*W*9."""
    return sum(2 * k * c * s * s * 9 for (c, k, s, _) in layers)


def algorithmic_bytes_per_image(esize, layers=VGG16_CONV):
    """Sum over layers of (input + output) activation bytes for one image (filters are batch independent)."""
    total = 0
    for (c, k, s, pool) in layers:
        o = s // 2 if pool else s
        total += (c * s * s + k * o * o) * esize
    return total


def winograd_gemm_flops_per_image(wino=4, layers=VGG16_CONV):
    """FLOPs of the tile GEMMs: 2 * a^2 * tiles * C * K, tiles = ceil(H/m)^2 (unpadded)."""
    a = wino + 2
    return sum(2 * a * a * math.ceil(s / wino) ** 2 * c * k for (c, k, s, _) in layers)


def kernel_model(batch, dtype="bf16", wino=4, layers=VGG16_CONV, layout="NHWC", forced_wino=False):
    """Algorithmic bytes and flops of one forward pass per kernel class, following the engine's per-layer choice
    for NHWC: C <= 3 (no pool): thin-input direct kernel; BF16 with C a multiple of 64 and (C <= 256, an image
    smaller than 28 x 28, fewer than 4 * 784 pixels in the batch, or NCHW tensors): direct tensor-core kernel; other tensor-core layers with C <= 128: row-fused tile GEMM
    (products Z, a*m planes, half for bf16); otherwise the plain tile GEMM (products M, a*a planes of floats, or of 3-byte values where the CTA-pair kernel
    writes them for an NHWC result)."""
    a, m = wino + 2, wino
    s_io = 2 if dtype == "bf16" else 4
    out = {k: {"bytes": 0, "flops": 0} for k in ("input_transform", "tile_gemm_plain", "tile_gemm_rowfused",
                                                 "output_transform", "direct_thin_input", "direct_tensor_core")}
    for (c, k, s, pool) in layers:
        o = s // 2 if pool else s
        if c <= 3 and not pool and not forced_wino:
            out["direct_thin_input"]["bytes"] += batch * (c * s * s + k * s * s) * s_io
            out["direct_thin_input"]["flops"] += batch * 2 * k * c * s * s * 9
            continue
        direct = (dtype == "bf16" and c % 64 == 0 and k % 8 == 0 and
                  (c <= 256 or s * s < 28 * 28 or batch * s * s < 4 * 28 * 28 or layout == "NCHW")) or \
                 (dtype == "tf32" and c % 32 == 0 and c <= 256 and k % 16 == 0 and k >= 64)
        if direct and not forced_wino:      # other layouts reach the same kernel through NHWC staging
            out["direct_tensor_core"]["bytes"] += batch * (c * s * s + k * o * o) * s_io
            out["direct_tensor_core"]["flops"] += batch * 2 * k * c * s * s * 9
            continue
        tiles = batch * math.ceil(s / m) ** 2
        cp, kq = math.ceil(c / 8) * 8, math.ceil(k / 8) * 8
        split = dtype == "fp32x3"      # V stays plain FP32 and is split into TF32 head + tail inside the tile GEMM
        v_bytes = a * a * tiles * cp * s_io
        fused = dtype in ("tf32", "bf16") and c <= 128
        # wide tensor-core layers with an NHWC result move the raw products in 3 bytes (CTA-pair tile GEMM, csrc/gemm_tc_pair.cu)
        m24 = (not fused and dtype in ("tf32", "bf16") and layout == "NHWC" and k >= 256 and k % 2 == 0 and cp >= 512 and
               kq % 16 == 0 and tiles >= 256)
        p_bytes = (a * m * tiles * kq * (2 if dtype == "bf16" else 4)) if fused else a * a * tiles * kq * (3 if m24 else 4)
        out["input_transform"]["bytes"] += batch * c * s * s * s_io + v_bytes
        g = out["tile_gemm_rowfused" if fused else "tile_gemm_plain"]
        g["bytes"] += v_bytes + p_bytes
        g["flops"] += 2 * a * a * tiles * c * k * (3 if split else 1)     # executed tensor-core flops
        out["output_transform"]["bytes"] += p_bytes + batch * k * o * o * s_io
    return out


class VGG16ConvStack:
    """The 13-layer stack for a fixed batch size, layout and dtype."""

    def __init__(self, batch, layout="NHWC", dtype="bf16", wino=0, seed=0xC0DE0040, device="cuda", layers=VGG16_CONV,
                 slab_images=0):
        self.batch, self.layout, self.dtype = batch, layout, dtype
        self.layers = list(layers)
        self.device = torch.device(device)
        self.io_dtype = torch.bfloat16 if dtype == "bf16" else torch.float32
        ws_bytes = 0
        for (c, k, s, pool) in self.layers:
            d = make_desc(batch, c, s, s, k, layout, None, dtype, 1, wino, True, True, pool, 0, slab_images)
            ws_bytes = max(ws_bytes, _lib.lib().wino_conv_workspace_bytes(ctypes.byref(d)))
        self.workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=self.device)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.convs, self.weights, self.biases = [], [], []
        max_act = 0
        for (c, k, s, pool) in self.layers:
            conv = WinoConv(batch, c, s, s, k, layout=layout, dtype=dtype, wino=wino, relu=True, bias=True, pool=pool,
                            slab_images=slab_images, device=device, workspace=self.workspace)
            w_kcrs = torch.randn((k, c, 3, 3), generator=gen) * math.sqrt(2.0 / (9 * c))
            b = torch.randn(k, generator=gen) * 0.01
            perm = {0: (0, 1, 2, 3), 1: (0, 2, 3, 1), 2: (1, 2, 3, 0)}[conv.desc.layout_in]
            w_l = w_kcrs.permute(perm).contiguous().to(self.io_dtype).to(self.device)
            b = b.to(self.device)
            conv.set_filter(w_l, b)
            self.convs.append(conv)
            self.weights.append(w_kcrs)
            self.biases.append(b)
            o = s // 2 if pool else s
            max_act = max(max_act, batch * k * o * o)
        self.act = [torch.empty(max_act, dtype=self.io_dtype, device=self.device) for _ in range(2)]
        c0, _, s0, _ = self.layers[0]
        self.in_shape = act_shape(layout, batch, c0, s0, s0)
        self.out_shape = self.convs[-1].out_shape
        self.launches_per_forward = None

    def forward(self, x):
        """x: input batch in `layout` (device tensor of in_shape).  Returns a view into an internal buffer."""
        cur = x
        for i, conv in enumerate(self.convs):
            out = self.act[i % 2][: math.prod(conv.out_shape)].view(conv.out_shape)
            conv(cur, out=out)
            cur = out
        return cur

    __call__ = forward

    def capture(self, x, prologue=None):
        """Record one forward pass over the fixed input buffer x into a CUDA graph (the 13-layer chain is short enough
        for launch gaps to show).  Runs one eager pass first: per-device set-up done on a kernel's first call cannot be
        captured.  `prologue`, if given, is called at the head of the captured region (the benchmark's L2 flush).
        Returns (graph, output view); graph.replay() recomputes the output from the current contents of x."""
        self.forward(x)
        torch.cuda.synchronize()
        before = _lib.lib().wino_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            if prologue is not None:
                prologue()
            y = self.forward(x)
        self.launches_per_forward = _lib.lib().wino_launch_count() - before
        return graph, y
