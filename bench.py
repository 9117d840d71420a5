#!/usr/bin/env python
"""Benchmark of the hot path: the VGG-16 convolution stack (13 3x3 convolutions with fused bias + ReLU, 2x2
max-pool fused at the five block ends) on synthetic data.

    python bench.py --gpus N --steps K --warmup W [--dtype bf16|tf32|fp32|fp32x3] [--layout NHWC|NCHW|CHWN]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...      (N > 1)
    python bench.py --impl reference ...        the CPU arm: the direct-convolution oracle on the host cores

One step = one forward pass of the stack over the batch.  The workload is ONE seeded batch of --batch images
(default 256) whatever the number of GPUs: the batch dimension is sharded contiguously over the ranks (256 / 128 /
64 / 32 images per GPU at 1 / 2 / 4 / 8 GPUs), weights are replicated, no collective sits on the data path, and the
job is strong-scaled.  --weak keeps --batch images on EVERY GPU instead (global batch N x --batch).
The timed region holds steps x inner passes (inner is chosen so that the region lasts about two seconds and the
power-capped clock is what gets measured); `ms_per_step` is the time of one pass.
Prints ONE JSON line on rank 0.
"""
import argparse
import glob
import json
import math
import os
import re
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "vgg16_conv_stack_images_per_s"
UNIT = "images/s"
L2_BYTES = 126 << 20             # the inputs of consecutive passes together exceed this (1.25x)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--inner", type=int, default=0, help="passes per timed step; 0 = as many as make the timed region last about 2 s")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "tf32", "fp32", "fp32x3"])
    ap.add_argument("--layout", default="NHWC", choices=["NHWC", "NCHW", "CHWN"])
    ap.add_argument("--batch", type=int, default=256, help="images per step over all GPUs (per GPU with --weak)")
    ap.add_argument("--weak", action="store_true", help="weak scaling: --batch images on every GPU")
    ap.add_argument("--wino", type=int, default=0, choices=[0, 2, 4])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cudnn-baseline", action="store_true", help="per-layer table without the cuDNN column")
    ap.add_argument("--no-layer-table", action="store_true", help="skip the per-layer table (ours and cuDNN) after the timed region")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--gather", action="store_true",
                    help="after the timed region, all-gather the final outputs over NCCL and check them bit for bit against the whole batch run on rank 0")
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

    def mark(self):
        """Samples taken from now on belong to the timed region."""
        self.first = len(self.lines)

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
        for line in self.lines[getattr(self, "first", 0):]:
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
    config = workload_config(args, args.gpus, None)
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
        images, config["global_batch"])
    emit(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True,
        "scaling": "weak" if args.weak else "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no C/C++ CPU convolution (its ground truth is a numpy triple loop); this arm times the "
                "C++ restatement of that loop, oracle/wino_ref.cpp"}))


def workload_config(args, world, inner, rotation=None):
    global_batch = args.batch * world if args.weak else args.batch
    return {"workload": "VGG-16 conv stack forward: 13 3x3 pad-1 convs 64,64|128,128|256x3|512x3|512x3, input 3x224x224, "
                        "bias+ReLU after each conv, 2x2 max-pool after each block",
            "global_batch": global_batch,
            "per_gpu_batch": args.batch if args.weak else [global_batch // world + (1 if r < global_batch % world else 0) for r in range(world)],
            "layout": args.layout,
            "parallelism": "batch-sharded x%d, no collective on the data path" % world,
            "init": "He-normal weights, bias N(0,0.01), input U[-1,1], seeded",
            "l2": "inputs larger than the L2: consecutive passes read %s distinct device copies of the batch in turn (together 1.25x "
                  "the 126 MB L2 or more), and every pass streams its activations (several times the L2) in between; the "
                  "end-to-end passes read inputs freshly copied from the host" % (rotation if rotation else "several"),
            "passes_per_timed_step": inner,
            "launch": "host launches" if getattr(args, "no_graph", False) else "one CUDA graph replay per pass"}


# ---- DRAM traffic from the committed ncu summaries --------------------------------------------------------
def profile_traffic_ratio(kernels, dtype, layout):
    """dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the captured launches, read from
    profiles/ncu_<kernel>_*.md (each captured launch there states its DRAM bytes and an `algorithmic_bytes` row).
    Returns (ratio, note) or (None, why)."""
    tag = "_%s_%s_" % (dtype, layout.lower())
    dram = alg = 0.0
    used = []
    for kernel in kernels:
        for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "ncu_%s_*%s*.md" % (kernel, tag)))):
            text = open(path).read()
            for block in text.split("## captured launch")[1:]:
                rd = re.search(r"dram__bytes_read\.sum \| ([0-9.]+) (\w+)", block)
                wr = re.search(r"dram__bytes_write\.sum \| ([0-9.]+) (\w+)", block)
                ab = re.search(r"algorithmic_bytes \| ([0-9]+)", block)
                if not (rd and wr and ab):
                    continue
                scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
                dram += float(rd.group(1)) * scale.get(rd.group(2), 1.0) + float(wr.group(1)) * scale.get(wr.group(2), 1.0)
                alg += float(ab.group(1))
                if os.path.basename(path) not in used:
                    used.append(os.path.basename(path))
    if alg <= 0:
        return None, "no ncu summary under profiles/ states DRAM and algorithmic bytes for %s (%s %s)" % ("+".join(kernels), dtype, layout)
    return dram / alg, "DRAM bytes / algorithmic bytes = %.3f over the captured launches of %s" % (dram / alg, ", ".join(used))


# ---- per-layer table with cuDNN beside it --------------------------------------------------------------------
def layer_table(stack, args, batch):
    """Per distinct layer shape: this library's fused layer (conv + bias + ReLU (+ pool)) and cuDNN's convolution alone
    (torch.nn.functional.conv2d with cudnn.benchmark, i.e. cuDNN's own pick among its engines; channels_last for NHWC),
    both timed the same way: 3 warm-up calls, then 10 back-to-back calls between two CUDA events, L2 not flushed
    (activations of these layers are far larger than the L2 at batch 256).  Outside the timed region of the benchmark."""
    import torch
    import torch.nn.functional as F
    torch.backends.cudnn.benchmark = True
    torch.backends.cudnn.allow_tf32 = args.dtype == "tf32"
    torch.backends.cuda.matmul.allow_tf32 = False
    tdt = stack.io_dtype
    rows, seen, error = [], {}, None
    for i, (conv, (c, k, s, pool)) in enumerate(zip(stack.convs, stack.layers)):
        key = (c, k, s, bool(pool))
        if key in seen:
            rows.append(dict(seen[key], layer=i + 1))
            continue
        x = (torch.rand(stack_in_shape(args.layout, batch, c, s), device="cuda") * 2 - 1).to(tdt)
        out = torch.empty(conv.out_shape, dtype=tdt, device="cuda")

        def ours():
            conv(x, out=out)

        ours_ms = time_calls(ours)
        cudnn_ms = None
        if not args.no_cudnn_baseline and args.dtype != "fp32x3":
            try:
                if args.layout == "NHWC":
                    xc = x.permute(0, 3, 1, 2)                          # a channels_last view of the same bytes
                    wc = torch.randn(k, 3, 3, c, device="cuda").to(tdt).permute(0, 3, 1, 2)
                elif args.layout == "NCHW":
                    xc, wc = x, torch.randn(k, c, 3, 3, device="cuda").to(tdt)
                else:                                                   # cuDNN has no CHWN: it gets NCHW
                    xc = x.permute(3, 0, 1, 2).contiguous()
                    wc = torch.randn(k, c, 3, 3, device="cuda").to(tdt)
                cudnn_ms = time_calls(lambda: F.conv2d(xc, wc, padding=1))
                del xc, wc
            except RuntimeError as e:
                cudnn_ms = None
                error = error or str(e).splitlines()[0][:160]
        flops = 2.0 * batch * k * c * s * s * 9
        row = {"layer": i + 1, "shape": "%d->%d@%d%s" % (c, k, s, "+pool" if pool else ""), "ours_ms": round(ours_ms, 4),
               "ours_tflops": round(flops / ours_ms / 1e9, 1), "cudnn_conv_only_ms": None if cudnn_ms is None else round(cudnn_ms, 4),
               "ours_over_cudnn_speed": None if cudnn_ms is None else round(cudnn_ms / ours_ms, 3)}
        seen[key] = row
        rows.append(row)
        del x, out
        torch.cuda.empty_cache()
    return rows, error


def stack_in_shape(layout, n, c, s):
    return {"NCHW": (n, c, s, s), "NHWC": (n, s, s, c), "CHWN": (c, s, s, n)}[layout]


def time_calls(fn, warm=3, iters=10):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


# ---- GPU arm --------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch
    import cudnntest_b200 as cb
    from cudnntest_b200 import shard, vgg
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (libwino has no CPU path)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = cb.lib()
    peaks = load_peaks()

    # the batch: one seeded tensor for the whole job (strong scaling: this rank's contiguous slice of it)
    global_batch = args.batch * world if args.weak else args.batch
    if args.weak:
        lo, hi = rank * args.batch, (rank + 1) * args.batch
    else:
        lo, hi = shard.shard_range(global_batch, world, rank)
    my_batch = hi - lo
    if my_batch <= 0:
        raise SystemExit("rank %d has no images: --batch %d is smaller than the number of GPUs" % (rank, args.batch))
    stack = vgg.VGG16ConvStack(my_batch, layout=args.layout, dtype=args.dtype, wino=args.wino, seed=0xC0DE0040)   # same weights on every rank
    axis = shard.BATCH_AXIS[args.layout]

    def host_images(first, last):
        """Images [first, last) of the job's batch in the stack's layout; image i is generated from seed 1234 + i."""
        imgs = []
        for i in range(first, last):
            g = torch.Generator(device="cpu").manual_seed(1234 + i)
            imgs.append(torch.rand((3, 224, 224), generator=g) * 2 - 1)
        x = torch.stack(imgs)                                               # NCHW
        perm = {"NCHW": (0, 1, 2, 3), "NHWC": (0, 2, 3, 1), "CHWN": (1, 2, 3, 0)}[args.layout]
        return x.permute(perm).contiguous().to(stack.io_dtype)

    x_host = host_images(lo, hi).pin_memory()
    x_dev = x_host.cuda(non_blocking=True)
    y_host = torch.empty(stack.out_shape, dtype=stack.io_dtype).pin_memory()
    stream = torch.cuda.current_stream()
    # Inputs larger than the L2: the resident passes read `rotation` device copies of the batch in turn, so that no pass
    # finds its input in the L2 because the pass before it read the same bytes.  Copies 0 and 1 double as the two
    # input buffers of the end-to-end passes.
    x_bytes = x_dev.numel() * x_dev.element_size()
    rotation = max(2, min(64, int(math.ceil(1.25 * L2_BYTES / x_bytes))))
    x_bufs = [x_dev] + [x_dev.clone() for _ in range(rotation - 1)]

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def all_max(v):
        if dist is None:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(pass_fn, passes, finish=None):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record(stream)
        for _ in range(passes):
            pass_fn()
        if finish is not None:
            finish()               # work still in flight on other streams joins the timed stream before the stop event
        stop.record(stream)
        torch.cuda.synchronize()
        barrier()
        return all_max(start.elapsed_time(stop))

    # One pass = the 13 layers, replayed from a CUDA graph (one per input buffer) unless --no-graph is given.
    graphs = None
    if not args.no_graph:
        graphs = [stack.capture(b) for b in x_bufs]
    launch_counter = {"n": 0}
    turn = {"i": 0}

    def run_stack(which):
        """One forward pass over input buffer `which`.  Returns the output view."""
        if graphs is None:
            before = L.wino_launch_count()
            y = stack(x_bufs[which])
            launch_counter["n"] += L.wino_launch_count() - before
            return y
        graphs[which][0].replay()
        launch_counter["n"] += stack.launches_per_forward
        return graphs[which][1]

    def pass_resident():
        run_stack(turn["i"] % rotation)
        turn["i"] += 1

    # End-to-end pass: every pass copies ITS input batch from pinned host memory and its result back.  The copy of
    # pass i+1's input runs on a second stream into the other of two device buffers while pass i computes; the result
    # is moved aside on the device (a few microseconds) and leaves for the host on a third stream, so neither copy
    # sits between two passes on the compute stream.
    copy_stream, out_stream = torch.cuda.Stream(), torch.cuda.Stream()
    ready = [torch.cuda.Event(), torch.cuda.Event()]       # input buffer b holds the next batch
    freed = [torch.cuda.Event(), torch.cuda.Event()]       # the compute that read buffer b has been issued and finished
    y_stage = [torch.empty(stack.out_shape, dtype=stack.io_dtype, device="cuda") for _ in range(2)]
    staged = [torch.cuda.Event(), torch.cuda.Event()]      # y_stage[b] holds a pass's result
    landed = [torch.cuda.Event(), torch.cuda.Event()]      # ... and it has reached the host
    e2e_state = {"i": 0, "primed": False}

    def upload(b):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[b])
            x_bufs[b].copy_(x_host, non_blocking=True)
            ready[b].record(copy_stream)

    def pass_e2e():
        b = e2e_state["i"] & 1
        if not e2e_state["primed"]:
            freed[0].record(stream); freed[1].record(stream)
            landed[0].record(out_stream); landed[1].record(out_stream)
            upload(b)
            e2e_state["primed"] = True
        upload(b ^ 1)                      # next pass's input, overlapped with this pass's compute
        stream.wait_event(ready[b])
        y = run_stack(b)
        freed[b].record(stream)
        stream.wait_event(landed[b])       # the result that used this staging buffer two passes ago is on the host
        y_stage[b].copy_(y, non_blocking=True)
        staged[b].record(stream)
        with torch.cuda.stream(out_stream):
            out_stream.wait_event(staged[b])
            y_host.copy_(y_stage[b], non_blocking=True)
            landed[b].record(out_stream)
        e2e_state["i"] += 1

    def finish_e2e():
        stream.wait_event(landed[0]); stream.wait_event(landed[1])

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        pass_resident()
    cb.device_status()
    # passes per step: enough for a timed region of about two seconds (same number on every rank)
    inner = args.inner
    if inner <= 0:
        est = timed(pass_resident, 3) / 3.0
        inner = max(1, int(math.ceil(2000.0 / (max(est, 1e-3) * args.steps))))
    passes = args.steps * inner
    launch_counter["n"] = 0
    if rank == 0:
        sampler.mark()
    ms = timed(pass_resident, passes)
    launches = launch_counter["n"]
    clocks = sampler.stop() if rank == 0 else None
    cb.device_status()

    for _ in range(2):
        pass_e2e()
    ms_e2e = timed(pass_e2e, passes, finish_e2e)
    cb.device_status()

    # per-kernel-class device time: five more passes launched from the host, each kernel bracketed by CUDA events on its stream
    import ctypes
    prof_passes = 5
    stack(x_dev)
    L.wino_profile_enable(1)
    for i in range(prof_passes):
        stack(x_bufs[(i + 1) % rotation])
    stage_ms = (ctypes.c_float * 8)()
    stage_n = (ctypes.c_longlong * 8)()
    L.wino_profile_read(stage_ms, stage_n)
    L.wino_profile_enable(0)

    gather = None
    if args.gather and dist is not None:      # off the timed path: the only collective of the job
        y_mine = stack(x_dev).clone()
        y_all = shard.gather_outputs(y_mine, args.layout, global_batch)
        torch.cuda.synchronize()
        gather = {"shape": list(y_all.shape)}
        if rank == 0 and not args.weak:
            # Images are independent, so sharding must not change a single bit: the gathered result has to equal the same
            # shards run one after the other on this GPU alone.  The whole batch as ONE 256-image run is compared too; it may
            # differ in rounding where the engine picks another kernel for another batch size (512 channels at 28 x 28:
            # direct kernel for a handful of images, Winograd otherwise; float or 3-byte products by the number of tile
            # rows), so that comparison also reports the relative L2 distance.
            pieces = []
            for r in range(world):
                lo_r, hi_r = shard.shard_range(global_batch, world, r)
                st = stack if hi_r - lo_r == my_batch else vgg.VGG16ConvStack(hi_r - lo_r, layout=args.layout, dtype=args.dtype,
                                                                                wino=args.wino, seed=0xC0DE0040)
                pieces.append(st(host_images(lo_r, hi_r).cuda()).clone())
            y_seq = torch.cat(pieces, dim=axis)
            torch.cuda.synchronize()
            gather["equals_same_shards_on_one_gpu"] = bool(torch.equal(y_seq, y_all))
            del pieces, y_seq
            whole = vgg.VGG16ConvStack(global_batch, layout=args.layout, dtype=args.dtype, wino=args.wino, seed=0xC0DE0040)
            y_whole = whole(host_images(0, global_batch).cuda())
            torch.cuda.synchronize()
            gather["equals_whole_batch_on_one_gpu"] = bool(torch.equal(y_whole, y_all))
            d = (y_whole.float() - y_all.float()).double()
            gather["rel_l2_vs_whole_batch_on_one_gpu"] = float(d.norm() / y_whole.float().double().norm().clamp_min(1e-30))
            del whole, y_whole

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    ms_pass = ms / passes
    ms_pass_e2e = ms_e2e / passes
    value = global_batch / (ms_pass * 1e-3)
    e2e_value = global_batch / (ms_pass_e2e * 1e-3)
    # Roofline of the kernel class with the largest share of the pass.  Algorithmic bytes / flops per class come from
    # vgg.kernel_model (every layer's units summed per kernel class); the bound is whichever of bytes / HBM peak and
    # flops / tensor peak is the longer time.
    model = vgg.kernel_model(my_batch, args.dtype, args.wino or 4, layout=args.layout, forced_wino=bool(args.wino))
    classes = {"input_transform": 0, "tile_gemm_plain": 1, "output_transform": 2, "tile_gemm_rowfused": 4, "direct_thin_input": 5,
               "direct_tensor_core": 6}
    stage = {n: {"ms": float(stage_ms[i]) / prof_passes, "launches": int(stage_n[i]) // prof_passes} for n, i in classes.items()}
    dominant = max(classes, key=lambda n: stage[n]["ms"])
    half = 0.5 if args.dtype in ("tf32", "fp32x3") else 1.0
    tpeak, tpeak_sustained = peaks["tflops_burst"] * half, peaks["tflops_sustained"] * half
    byts, flops = model[dominant]["bytes"], model[dominant]["flops"]
    t_meas = max(stage[dominant]["ms"], 1e-9) * 1e-3
    t_hbm, t_tc = byts / (peaks["hbm_gbs"] * 1e9), flops / (tpeak * 1e12)
    in_kernel = {"NHWC": "input_transform_nhwc_tma", "NCHW": "input_transform_strip", "CHWN": "input_transform_batch"}[args.layout]
    out_kernel = {"NHWC": "output_transform_direct_x2", "NCHW": "output_transform_strip", "CHWN": "output_transform_batch"}[args.layout]
    kernel_names = {"input_transform": [in_kernel],
                    "tile_gemm_plain": [{"fp32": "gemm_ffma_kernel", "fp32x3": "gemm_tc_split_kernel"}.get(args.dtype, "gemm_tc_kernel")],
                    "output_transform": [out_kernel], "tile_gemm_rowfused": ["gemm_tc_z_kernel"],
                    "direct_thin_input": ["direct_small_c_kernel"], "direct_tensor_core": ["direct_tc2t_kernel", "direct_tc2_kernel"]}
    if t_hbm >= t_tc or args.dtype == "fp32":
        achieved = byts / t_meas / 1e9
        roofline = {"kernel": " + ".join(kernel_names[dominant]), "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                    "peak_source": peaks["source"] + " copy bandwidth"}
    else:
        achieved = flops / t_meas / 1e12
        roofline = {"kernel": " + ".join(kernel_names[dominant]), "bound": "tensor", "achieved": achieved, "peak": tpeak,
                    "unit": "TFLOP/s", "frac": achieved / tpeak, "frac_sustained": achieved / tpeak_sustained,
                    "peak_sustained": tpeak_sustained, "traffic": None,
                    "peak_source": peaks["source"] + " bf16 cuBLAS, burst (the class is timed kernel by kernel in host-launched passes); "
                                   "frac_sustained divides by the seconds-long figure" + (", both halved for tf32" if half < 1 else "")}
    if args.dtype == "fp32" and dominant == "tile_gemm_plain":
        roofline["note"] = ("the exact-FP32 tile GEMM is bound by the FP32 FMA pipe, which this object's hbm|tensor vocabulary does not "
                            "name: %.1f TFLOP/s of a nominal 74.4 (148 SMs x 128 lanes x 2 x 1.965 GHz)" % (flops / t_meas / 1e12))
    ratio, note = profile_traffic_ratio(kernel_names[dominant], args.dtype, args.layout)
    if ratio is not None:
        roofline["traffic"] = ratio * byts / max(stage[dominant]["launches"], 1)
    roofline["traffic_note"] = note + ("; applied to the algorithmic bytes per launch of this run" if ratio is not None else "")
    roofline["algorithmic_bytes_per_pass"] = byts
    roofline["algorithmic_flops_per_pass"] = flops
    roofline["launches_per_pass"] = stage[dominant]["launches"]
    roofline["ms_per_pass"] = round(stage[dominant]["ms"], 4)
    roofline["per_class"] = {
        n: {"ms": round(stage[n]["ms"], 4), "launches": stage[n]["launches"],
            "hbm_frac": round(model[n]["bytes"] / max(stage[n]["ms"], 1e-9) / 1e6 / peaks["hbm_gbs"], 4),
            "tensor_frac": round(model[n]["flops"] / max(stage[n]["ms"], 1e-9) / 1e9 / tpeak, 4)}
        for n in classes if stage[n]["launches"]}

    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm, "inner": inner,
        "timed_passes": passes, "timed_region_ms": ms, "ms_per_step": ms_pass, "higher_is_better": True,
        "scaling": "weak" if args.weak else "strong", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic", "config": workload_config(args, world, inner, rotation),
        "tflops_direct_equivalent": vgg.direct_flops_per_image() * value / 1e12,
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": x_host.numel() // my_batch * global_batch * x_host.element_size(),
                "d2h_bytes_per_step": y_host.numel() // my_batch * global_batch * y_host.element_size(), "ms_per_step": ms_pass_e2e},
        "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
    }
    if clocks and clocks.get("sm_mhz"):
        out["ms_x_mhz_per_step"] = ms_pass * clocks["sm_mhz"]
    if gather is not None:
        out["gather"] = gather
    if world == 1 and not args.no_layer_table:
        # baselines measured in this process, outside the timed region
        rows, err = layer_table(stack, args, my_batch)
        have = [r for r in rows if r["cudnn_conv_only_ms"] is not None]
        out["baselines"] = {"cudnn": {
            "how": "torch.nn.functional.conv2d, cudnn.benchmark=True (cuDNN %s), %s, convolution alone; ours = the fused layer "
                   "(conv + bias + ReLU (+ 2x2 pool)); 10 back-to-back calls between CUDA events after 3 warm-ups"
                   % (torch.backends.cudnn.version(), "channels_last" if args.layout == "NHWC" else "NCHW"),
            "per_layer": rows,
            "ours_sum_ms": round(sum(r["ours_ms"] for r in rows), 4),
            "cudnn_conv_only_sum_ms": round(sum(r["cudnn_conv_only_ms"] for r in have), 4) if len(have) == len(rows) else None,
            "layers_at_or_above_cudnn": sum(1 for r in have if r["ours_over_cudnn_speed"] >= 1.0), "layers": len(rows)}}
        if err:
            out["baselines"]["cudnn"]["error"] = err
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
