"""Batch sharding across GPUs: the only multi-GPU mechanism of the convolution path.

Images are independent through convolution, bias, ReLU and pooling, so the batch dimension is partitioned
contiguously over the ranks (one process per GPU), weights are replicated, and no collective sits on the
data path.  The reference is single-GPU (hard-coded ``cudaSetDevice(1)``, comparison/layoutCompare.cu:33-34);
its ``bat4Conv`` argument is the only batch notion.  ``gather_outputs`` is the optional final all-gather of the
per-rank results (off the timed path).
"""
import torch

BATCH_AXIS = {"NCHW": 0, "NHWC": 0, "CHWN": 3}


def shard_range(total, world, rank):
    """Contiguous [start, stop) of `total` images for `rank` of `world`; the first total % world ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank %d of %d" % (rank, world))
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_tensor(x, layout, world, rank):
    """This rank's images of an activation tensor stored in `layout` (a contiguous copy)."""
    axis = BATCH_AXIS[layout]
    lo, hi = shard_range(x.shape[axis], world, rank)
    return x.narrow(axis, lo, hi - lo).contiguous()


def gather_outputs(y_local, layout, total, group=None):
    """All-gather the per-rank outputs back into the full batch (every rank gets the whole tensor)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    axis = BATCH_AXIS[layout]
    sizes = [shard_range(total, world, r) for r in range(world)]
    pieces = []
    for (lo, hi) in sizes:
        shape = list(y_local.shape)
        shape[axis] = hi - lo
        pieces.append(torch.empty(shape, dtype=y_local.dtype, device=y_local.device))
    if len({hi - lo for lo, hi in sizes}) == 1:
        dist.all_gather(pieces, y_local.contiguous(), group=group)
    else:   # ragged shards: one broadcast per rank
        rank = dist.get_rank(group)
        for r, p in enumerate(pieces):
            if r == rank:
                p.copy_(y_local)
            dist.broadcast(p, src=dist.get_global_rank(group, r) if group is not None else r, group=group)
    return torch.cat(pieces, dim=axis)
