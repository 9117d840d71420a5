"""Single-layer benchmark configurations: every variant is timed on seeded synthetic tensors and reported as
direct-convolution-equivalent TFLOP/s, images/s and as a fraction of the roofline that bounds the fused layer.

    python -m cudnntest_b200.configs [--iters 20] [--config 0 1 2 3]

The four configurations are the single-layer shapes the reference's harnesses are driven with
(comparison/layoutCompare.cu:41-82 layers 6, 8, 9 and the 64 -> 64 case of layoutTest): all 3x3, stride 1, pad 1.

  0  N=8,   C=K=64,  56x56, FP32 (and FP32X3), NCHW, no bias / ReLU
  1  N=64,  C=K=256, 56x56, {FP32, FP32X3, TF32, BF16} x {NCHW, NHWC, CHWN}, bias + ReLU
  2  N=64,  C=K=512, 28x28, {F(2x2,3x3), F(4x4,3x3)} x {BF16, FP32, FP32X3} x {NHWC, CHWN}
  3  N=128, C=K=512, 14x14, BF16, NCHW, bias + ReLU

One JSON line per variant.  Figures: flops = 2 N K C H W 9 (direct-convolution equivalent); bytes = (x + w + y) in
the storage type (+ 4 K for the bias); roofline time = max(bytes / HBM bandwidth, arithmetic / peak) where the
arithmetic is what the chosen kernel really executes (the Winograd tile GEMM's 2 a^2 T C K, or the direct flops) and
the peak is the measured BF16 tensor rate (half of it for TF32; FP32X3 executes three TF32 passes) or the nominal
FP32 FFMA rate.  Inputs smaller than
the L2 are evicted by rewriting a 256 MiB buffer before every timed call.
"""
import argparse
import json
import math
import os

import torch

from . import _lib
from .conv import WinoConv, act_shape, device_status, filter_shape

CONFIGS = {
    0: dict(n=8, c=64, k=64, s=56, bias=False, relu=False, variants=[("fp32", "NCHW", 0), ("fp32x3", "NCHW", 0)]),
    1: dict(n=64, c=256, k=256, s=56, bias=True, relu=True,
            variants=[(dt, lo, 0) for dt in ("fp32", "fp32x3", "tf32", "bf16") for lo in ("NCHW", "NHWC", "CHWN")]),
    2: dict(n=64, c=512, k=512, s=28, bias=False, relu=False,
            variants=[(dt, lo, wino) for wino in (2, 4) for dt in ("bf16", "fp32", "fp32x3") for lo in ("NHWC", "CHWN")]),
    3: dict(n=128, c=512, k=512, s=14, bias=True, relu=True, variants=[("bf16", "NCHW", 0)]),
}

FFMA_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12      # 148 SMs x 128 FP32 lanes x 2 flops x max SM clock


def load_peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def engine_runs_winograd(dtype, layout, n, c, k, s, wino):
    """Mirror of the library's per-layer choice for these shapes (C a multiple of 64, K a multiple of 16)."""
    if wino or dtype in ("fp32", "fp32x3"):
        return True
    if dtype == "bf16":
        return not (c <= 256 or s * s < 28 * 28 or n * s * s < 4 * 28 * 28 or layout == "NCHW")
    return c > 256      # tf32


def run_variant(cfg_id, cfg, dtype, layout, wino, iters, peaks, flush):
    n, c, k, s = cfg["n"], cfg["c"], cfg["k"], cfg["s"]
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    es = 2 if dtype == "bf16" else 4
    gen = torch.Generator(device="cpu").manual_seed(0xC0DE0000 + 16 * cfg_id)
    x = (torch.rand(act_shape(layout, n, c, s, s), generator=gen) * 2 - 1).to(tdt).cuda()
    w = (torch.randn(filter_shape(layout, k, c), generator=gen) * math.sqrt(2.0 / (9 * c))).to(tdt).cuda()
    b = (torch.randn(k, generator=gen) * 0.01).cuda() if cfg["bias"] else None
    conv = WinoConv(n, c, s, s, k, layout=layout, dtype=dtype, wino=wino, relu=cfg["relu"], bias=cfg["bias"])
    conv.set_filter(w, b)
    y = torch.empty(conv.out_shape, dtype=tdt, device="cuda")
    for _ in range(5):
        conv(x, out=y)
    torch.cuda.synchronize()
    device_status()
    times = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        conv(x, out=y)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    device_status()
    times.sort()
    ms = times[len(times) // 2]
    flops = 2.0 * n * k * c * s * s * 9
    byts = (n * c * s * s + 9 * k * c + n * k * s * s) * es + (4 * k if cfg["bias"] else 0)
    winograd = engine_runs_winograd(dtype, layout, n, c, k, s, wino)
    m = wino or 4
    arithmetic = 2.0 * (m + 2) ** 2 * n * math.ceil(s / m) ** 2 * c * k if winograd else flops
    if dtype == "fp32x3":
        arithmetic *= 3     # three TF32 products rebuild one FP32 product
    peak = {"bf16": peaks["bf16_tflops"], "tf32": peaks["bf16_tflops"] / 2, "fp32x3": peaks["bf16_tflops"] / 2,
            "fp32": FFMA_TFLOPS_NOMINAL}[dtype]
    t_hbm, t_math = byts / (peaks["hbm_gbs"] * 1e9), arithmetic / (peak * 1e12)
    roof_ms = max(t_hbm, t_math) * 1e3
    return {"config": cfg_id, "n": n, "c": c, "k": k, "h": s, "dtype": dtype, "layout": layout,
            "kernel": ("winograd F(%dx%d,3x3)" % (m, m)) if winograd else "direct (implicit GEMM)",
            "ms": round(ms, 4), "ms_min": round(times[0], 4), "tflops_direct_equivalent": round(flops / ms / 1e9, 1),
            "images_per_s": round(n / ms * 1e3, 1), "algorithmic_bytes": byts,
            "roofline": {"bound": "hbm" if t_hbm >= t_math else ("tensor" if dtype != "fp32" else "ffma"),
                         "roofline_ms": round(roof_ms, 4), "frac": round(roof_ms / ms, 3),
                         "hbm_gbs": peaks["hbm_gbs"], "peak_tflops": round(peak, 1),
                         "peaks": peaks["source"] + (" (FP32 FFMA: nominal)" if dtype == "fp32" else "")}}


def measure_library_peaks(n=8192, reps=10):
    """cuBLAS rates the peaks file does not hold, measured the way its BF16 figure was (torch.matmul, n^3, burst of
    `reps` calls between two CUDA events): TF32 tensor-core GEMM and FP32 SGEMM on float operands."""
    a = torch.randn((n, n), device="cuda")
    b = torch.randn((n, n), device="cuda")
    out = {}
    old = torch.backends.cuda.matmul.allow_tf32
    try:
        for name, allow in (("tf32_tflops", True), ("fp32_sgemm_tflops", False)):
            torch.backends.cuda.matmul.allow_tf32 = allow
            for _ in range(3):
                a @ b
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                a @ b
            e1.record()
            torch.cuda.synchronize()
            out[name] = round(2.0 * n ** 3 * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12, 1)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--config", type=int, nargs="*", default=[0, 1, 2, 3])
    ap.add_argument("--library-peaks", action="store_true",
                    help="print cuBLAS TF32 and FP32 SGEMM TFLOP/s of this GPU (one JSON line) and exit")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: this library has no CPU path")
    if args.library_peaks:
        print(json.dumps(dict(measure_library_peaks(), what="torch.matmul 8192^3, float operands, burst of 10")))
        return
    _lib.lib()
    peaks = load_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for cid in args.config:
        cfg = CONFIGS[cid]
        for (dtype, layout, wino) in cfg["variants"]:
            print(json.dumps(run_variant(cid, cfg, dtype, layout, wino, args.iters, peaks, flush)), flush=True)


if __name__ == "__main__":
    main()
