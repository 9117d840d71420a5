"""Host-side pieces of bench.py that need no GPU: the shard sizes the JSON line reports and the DRAM-traffic figure
read from the committed ncu summaries."""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench  # noqa: E402


def _args(**kw):
    base = dict(batch=256, weak=False, layout="NHWC", no_graph=False)
    base.update(kw)
    return argparse.Namespace(**base)


def test_strong_scaling_shards_one_batch():
    for world in (1, 2, 4, 8):
        cfg = bench.workload_config(_args(), world, 10, 3)
        assert cfg["global_batch"] == 256 and sum(cfg["per_gpu_batch"]) == 256 and len(cfg["per_gpu_batch"]) == world
    cfg = bench.workload_config(_args(batch=10), 4, 1, 2)
    assert cfg["per_gpu_batch"] == [3, 3, 2, 2]
    weak = bench.workload_config(_args(weak=True), 8, 1, 2)
    assert weak["global_batch"] == 2048 and weak["per_gpu_batch"] == 256


def test_traffic_ratio_comes_from_the_profiles():
    ratio, note = bench.profile_traffic_ratio(["direct_tc2t_kernel", "direct_tc2_kernel"], "bf16", "NHWC")
    assert ratio is not None and 0.3 < ratio < 3.0
    assert "ncu_direct_tc2t_kernel" in note and "ncu_direct_tc2_kernel" in note
    for kernel in ("gemm_tc_pair_kernel", "input_transform_nhwc_tma", "output_transform_direct_x2", "direct_small_c_kernel"):
        r, _ = bench.profile_traffic_ratio([kernel], "bf16", "NHWC")
        assert r is not None and 0.3 < r < 3.0, kernel
    none, why = bench.profile_traffic_ratio(["no_such_kernel"], "bf16", "NHWC")
    assert none is None and "no ncu summary" in why
