"""Batch sharding over two ranks on the CPU (gloo): ranges, per-layout slicing and the final gather.

The compute in each rank is the CPU oracle's convolution (no GPU here); what is under test is the host logic of
cudnntest_b200/shard.py that the multi-GPU benchmark uses."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, layout, total, results):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import oracle
    from cudnntest_b200 import shard
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        x = rng.uniform(-1, 1, (total, 4, 6, 6)).astype(np.float32)
        w = rng.standard_normal((5, 4, 3, 3)).astype(np.float32)
        xl = torch.from_numpy(oracle.to_layout(x, layout))
        mine = shard.shard_tensor(xl, layout, world, rank)
        lo, hi = shard.shard_range(total, world, rank)
        assert mine.shape[shard.BATCH_AXIS[layout]] == hi - lo
        y_local = torch.from_numpy(oracle.conv_f64(mine.numpy(), oracle.filter_to_layout(w, layout), relu=True, layout=layout))
        y_all = shard.gather_outputs(y_local, layout, total)
        ref = oracle.conv_f64(oracle.to_layout(x, layout), oracle.filter_to_layout(w, layout), relu=True, layout=layout)
        results[rank] = bool(np.array_equal(y_all.numpy(), ref))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout,total", [("NHWC", 6), ("NCHW", 5), ("CHWN", 7)])
def test_two_rank_shard_and_gather(layout, total):
    world = 2
    port = 29500 + (os.getpid() + total) % 2000
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, layout, total, results), nprocs=world, join=True)
        assert results.get(0) is True and results.get(1) is True


def test_shard_ranges_cover_batch():
    from cudnntest_b200.shard import shard_range
    for total in (0, 1, 7, 256):
        for world in (1, 2, 4, 8):
            spans = [shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(hi - lo for lo, hi in spans) - min(hi - lo for lo, hi in spans) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)
