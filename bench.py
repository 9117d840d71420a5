#!/usr/bin/env python
"""Benchmark of the hot path: the VGG-16 convolution stack (13 Winograd 3x3 convolutions with fused
bias + ReLU, 2x2 max-pool fused at the five block ends) on synthetic data.

    python bench.py --gpus N --steps K --warmup W [--dtype bf16|tf32|fp32|fp32x3] [--layout NHWC|NCHW|CHWN]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...      (N > 1)
    python bench.py --impl reference ...        the CPU arm: the direct-convolution oracle on the host cores

One step = one forward pass of the stack over one batch.  The batch dimension shards across GPUs with
no data-path collective (every rank runs its own images with replicated weights); per-GPU batch is fixed
at --batch (default 256), so the job is weak-scaled and `value` is the aggregate images/s.
Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "vgg16_conv_stack_images_per_s"
UNIT = "images/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "tf32", "fp32", "fp32x3"])
    ap.add_argument("--layout", default="NHWC", choices=["NHWC", "NCHW", "CHWN"])
    ap.add_argument("--batch", type=int, default=256, help="images per GPU per step")
    ap.add_argument("--wino", type=int, default=0, choices=[0, 2, 4])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--gather", action="store_true", help="after the timed region, all-gather the final outputs over NCCL once")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU time of the cpu_baseline sample")
    return ap.parse_args()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


# ---- clocks -------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # nvidia-smi takes a moment to initialise NVML (and holds driver locks while it does): let it deliver its
            # first sample before anything is timed
            t0 = time.time()
            while not self.lines and time.time() - t0 < 10.0 and self.proc.poll() is None:
                time.sleep(0.05)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(power)}


# ---- CPU arm --------------------------------------------------------------------------------------------
def cpu_stack_images_per_s(layout, images, repeats=1):
    """Times the oracle's float32 direct convolution (all host threads) over the 13-layer stack."""
    import numpy as np
    import oracle
    from cudnntest_b200.vgg import VGG16_CONV
    rng = np.random.default_rng(0xC0DE0040)
    x = oracle.to_layout(rng.uniform(-1, 1, (images, 3, 224, 224)).astype(np.float32), layout)
    ws, bs = [], []
    for (c, k, s, pool) in VGG16_CONV:
        ws.append(oracle.filter_to_layout((rng.standard_normal((k, c, 3, 3)) * np.sqrt(2.0 / (9 * c))).astype(np.float32), layout))
        bs.append((rng.standard_normal(k) * 0.01).astype(np.float32))
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        cur = x
        for (c, k, s, pool), w, b in zip(VGG16_CONV, ws, bs):
            cur = oracle.conv_f32(cur, w, bias=b, relu=True, pool=pool, layout=layout)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return images / best, best


def cpu_baseline(layout, target_seconds):
    import oracle
    rate, dt = cpu_stack_images_per_s(layout, 1)
    images = int(max(1, min(64, target_seconds / max(dt, 1e-3))))
    if images > 1:
        rate, dt = cpu_stack_images_per_s(layout, images)
    return {"value": rate, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
            "sample": "%d image(s) through all 13 layers, float32 direct convolution (oracle/wino_ref.cpp, OpenMP), "
                      "%.1f s" % (images, dt)}


def run_reference(args, rank):
    if rank != 0:
        return
    import oracle
    oracle.build()
    oracle.set_num_threads(len(os.sched_getaffinity(0)))    # all host cores, whatever the launcher put in OMP_NUM_THREADS
    config = workload_config(args)
    rate, dt = cpu_stack_images_per_s(args.layout, 1)       # sizing probe
    images = int(max(1, min(16, 20.0 / max(dt, 1e-3) / max(args.steps + args.warmup, 1))))
    for _ in range(args.warmup):
        cpu_stack_images_per_s(args.layout, images)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_stack_images_per_s(args.layout, images)
    total = time.perf_counter() - t0
    value = images * args.steps / total
    sample = "each step = %d image(s) through all 13 layers on the host cores (bounded sample of the %d-image batch)" % (
        images, args.batch)
    emit(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no C/C++ CPU convolution (its ground truth is a numpy triple loop); this arm times the "
                "C++ restatement of that loop, oracle/wino_ref.cpp"}))


def workload_config(args):
    return {"workload": "VGG-16 conv stack forward: 13 3x3 pad-1 convs 64,64|128,128|256x3|512x3|512x3, input 3x224x224, "
                        "bias+ReLU after each conv, 2x2 max-pool after each block",
            "per_gpu_batch": args.batch, "global_batch": args.batch * args.gpus, "layout": args.layout,
            "parallelism": "batch-sharded x%d, no collective" % args.gpus,
            "init": "He-normal weights, bias N(0,0.01), input U[-1,1], seeded",
            "l2": "256 MiB buffer rewritten between timed iterations",
            "launch": "host launches" if getattr(args, "no_graph", False) else "one CUDA graph replay per step"}


# ---- GPU arm --------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch
    import cudnntest_b200 as cb
    from cudnntest_b200 import vgg
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (libwino has no CPU path)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = cb.lib()
    peaks = load_peaks()

    stack = vgg.VGG16ConvStack(args.batch, layout=args.layout, dtype=args.dtype, wino=args.wino, seed=0xC0DE0040 + rank)
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    x_host = (torch.rand(stack.in_shape, generator=gen) * 2 - 1).to(stack.io_dtype).pin_memory()
    x_dev = x_host.cuda(non_blocking=True)
    y_host = torch.empty(stack.out_shape, dtype=stack.io_dtype).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(step_fn, steps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record(stream)
        for _ in range(steps):
            flush.zero_()
            step_fn()
        stop.record(stream)
        torch.cuda.synchronize()
        barrier()
        ms = start.elapsed_time(stop)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # The forward pass is replayed from a CUDA graph (one per input buffer) unless --no-graph is given.
    x_bufs = [torch.empty_like(x_dev), torch.empty_like(x_dev)]
    graphs = None
    if not args.no_graph:
        graphs = [stack.capture(b) for b in [x_dev] + x_bufs]
    launch_counter = {"n": 0}

    def run_stack(which):
        """which: 0 = resident input, 1 / 2 = the end-to-end input buffers.  Returns the output view."""
        if graphs is None:
            before = L.wino_launch_count()
            y = stack(([x_dev] + x_bufs)[which])
            launch_counter["n"] += L.wino_launch_count() - before
            return y
        graphs[which][0].replay()
        launch_counter["n"] += stack.launches_per_forward
        return graphs[which][1]

    def step_resident():
        run_stack(0)

    # End-to-end step: every step copies ITS input batch from pinned host memory and its result back.  The copy of
    # step i+1's input runs on a second stream into the other of two device buffers while step i computes.
    copy_stream = torch.cuda.Stream()
    ready = [torch.cuda.Event(), torch.cuda.Event()]       # input buffer b holds the next batch
    freed = [torch.cuda.Event(), torch.cuda.Event()]       # the compute that read buffer b has been issued and finished
    e2e_state = {"i": 0, "primed": False}

    def upload(b):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[b])
            x_bufs[b].copy_(x_host, non_blocking=True)
            ready[b].record(copy_stream)

    def step_e2e():
        b = e2e_state["i"] & 1
        if not e2e_state["primed"]:
            freed[0].record(stream); freed[1].record(stream)
            upload(b)
            e2e_state["primed"] = True
        upload(b ^ 1)                      # next step's input, overlapped with this step's compute
        stream.wait_event(ready[b])
        y = run_stack(1 + b)
        freed[b].record(stream)
        y_host.copy_(y, non_blocking=True)
        e2e_state["i"] += 1

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()            # samples run from here to the end of the timed region (warm-up included: same load)
    for _ in range(max(args.warmup, 3)):
        step_resident()
    cb.device_status()
    launch_counter["n"] = 0
    ms = timed(step_resident, args.steps)
    launches = launch_counter["n"]
    clocks = sampler.stop() if rank == 0 else None
    cb.device_status()

    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    cb.device_status()

    # per-stage device time of one more step, each kernel bracketed by events on its stream
    import ctypes
    L.wino_profile_enable(1)
    stack(x_dev)                   # launched from the host: the profiling events are not part of the captured graph
    stage_ms = (ctypes.c_float * 8)()
    stage_n = (ctypes.c_longlong * 8)()
    L.wino_profile_read(stage_ms, stage_n)
    L.wino_profile_enable(0)

    gathered = None
    if args.gather and dist is not None:      # optional, off the timed path: the only collective of the job
        from cudnntest_b200 import shard
        y_all = shard.gather_outputs(stack(x_dev).clone(), args.layout, args.batch * world)
        torch.cuda.synchronize()
        gathered = list(y_all.shape)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    images = args.batch * world
    value = images * args.steps / (ms * 1e-3)
    e2e_value = images * args.steps / (ms_e2e * 1e-3)
    # Roofline of the kernel class with the largest share of the step.  Algorithmic bytes / flops per launch set
    # come from vgg.kernel_model (every layer's units summed per kernel class); the bound is whichever of
    # bytes / HBM peak and flops / tensor peak is the longer time.
    model = vgg.kernel_model(args.batch, args.dtype, args.wino or 4, layout=args.layout, forced_wino=bool(args.wino))
    classes = {"input_transform": 0, "tile_gemm_plain": 1, "output_transform": 2, "tile_gemm_rowfused": 4, "direct_thin_input": 5,
               "direct_tensor_core": 6}
    stage = {n: {"ms": float(stage_ms[i]), "launches": int(stage_n[i])} for n, i in classes.items()}
    dominant = max(classes, key=lambda n: stage[n]["ms"])
    tpeak = peaks["tflops_sustained"] * (0.5 if args.dtype in ("tf32", "fp32x3") else 1.0)
    byts, flops = model[dominant]["bytes"], model[dominant]["flops"]
    t_meas = stage[dominant]["ms"] * 1e-3
    t_hbm, t_tc = byts / (peaks["hbm_gbs"] * 1e9), flops / (tpeak * 1e12)
    kernel_names = {"input_transform": "input_transform_nhwc_tma", "tile_gemm_plain": {"fp32": "gemm_ffma_kernel", "fp32x3": "gemm_tc_split_kernel"}.get(args.dtype, "gemm_tc_kernel"),
                    "output_transform": "output_transform_direct", "tile_gemm_rowfused": "gemm_tc_z_kernel",
                    "direct_thin_input": "direct_small_c_kernel", "direct_tensor_core": "direct_tc2t_kernel + direct_tc2_kernel"}
    if t_hbm >= t_tc or args.dtype == "fp32":
        achieved = byts / t_meas / 1e9
        roofline = {"kernel": kernel_names[dominant], "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"] + " copy bandwidth"}
    else:
        achieved = flops / t_meas / 1e12
        roofline = {"kernel": kernel_names[dominant], "bound": "tensor", "achieved": achieved, "peak": tpeak, "unit": "TFLOP/s",
                    "frac": achieved / tpeak, "traffic": None,
                    "peak_source": peaks["source"] + " sustained bf16 cuBLAS" + (" halved for tf32" if args.dtype in ("tf32", "fp32x3") else "")}
    if args.dtype == "fp32" and dominant == "tile_gemm_plain":
        roofline["note"] = ("the exact-FP32 tile GEMM is bound by the FP32 FMA pipe, which this object's hbm|tensor vocabulary does not "
                            "name: %.1f TFLOP/s of a nominal 74.4 (148 SMs x 128 lanes x 2 x 1.965 GHz)" % (flops / t_meas / 1e12))
    # DRAM traffic per launch: ncu's dram__bytes_read.sum + dram__bytes_write.sum of one captured launch of this kernel
    # (profiles/ncu_<kernel>_vgg16_bf16_nhwc_batch32.md) divided by that launch's algorithmic bytes, applied to the
    # average algorithmic bytes per launch here.  Reads match the algorithmic bytes; output still dirty in the 126 MB L2
    # when the captured launch ends is not in ncu's write count, hence ratios below 1.
    ncu_ratio = {"direct_tensor_core": 0.78, "tile_gemm_plain": 0.71, "output_transform": 0.93, "input_transform": 0.92,
                 "direct_thin_input": 0.73, "tile_gemm_rowfused": 0.88}
    if args.dtype == "bf16" and args.layout == "NHWC":
        roofline["traffic"] = ncu_ratio[dominant] * byts / max(stage[dominant]["launches"], 1)
        roofline["traffic_note"] = "bytes per launch = ncu DRAM/algorithmic ratio %.2f (batch-32 capture) x algorithmic bytes per launch" % ncu_ratio[dominant]
    roofline["algorithmic_bytes_per_step"] = byts
    roofline["algorithmic_flops_per_step"] = flops
    roofline["launches_per_step"] = stage[dominant]["launches"]
    roofline["ms_per_step"] = round(stage[dominant]["ms"], 4)
    roofline["per_class"] = {
        n: {"ms": round(stage[n]["ms"], 4), "launches": stage[n]["launches"],
            "hbm_frac": round(model[n]["bytes"] / max(stage[n]["ms"], 1e-9) / 1e6 / peaks["hbm_gbs"], 4),
            "tensor_frac": round(model[n]["flops"] / max(stage[n]["ms"], 1e-9) / 1e9 / tpeak, 4)}
        for n in classes if stage[n]["launches"]}

    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic", "config": workload_config(args),
        "tflops_direct_equivalent": vgg.direct_flops_per_image() * value / 1e12,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * x_host.element_size() * world,
                "d2h_bytes_per_step": y_host.numel() * y_host.element_size() * world, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
    }
    if gathered is not None:
        out["gathered_output_shape"] = gathered
    if world == 1 and not args.no_cpu_baseline:
        import oracle
        oracle.build()
        oracle.set_num_threads(len(os.sched_getaffinity(0)))
        out["cpu_baseline"] = cpu_baseline(args.layout, args.cpu_seconds)
    emit(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


_RESULT_FD = None


def emit(line):
    """Write the one result line to the process's real stdout."""
    if _RESULT_FD is None:
        print(line, flush=True)
    else:
        os.write(_RESULT_FD, (line + "\n").encode())


def main():
    global _RESULT_FD
    args = parse_args()
    # stdout carries exactly one JSON line: anything a library prints there (NCCL's version banner, for one) goes to stderr
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus %d needs torchrun with %d ranks (one process per GPU)" % (args.gpus, args.gpus))
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
