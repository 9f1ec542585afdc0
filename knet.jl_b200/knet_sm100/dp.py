"""Host-side rules of the data-parallel training step (one process per GPU).

Knet has no multi-GPU path; this is the batch-sharded step of the MLP benchmark: every rank
holds the same weights and optimizer state, takes a contiguous shard of the batch columns,
all-reduces (sum) each layer's gradient bucket as soon as it is final, and folds the 1/world
factor into the optimizer's read of the gradient.  The functions here are backend-agnostic
(NCCL on GPUs, gloo in the CPU tests).
"""
import os

import torch
import torch.distributed as dist


def init_from_env(backend):
    """Create the default process group from torchrun's environment; returns (rank, world)."""
    if "RANK" not in os.environ:
        return 0, 1
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if not dist.is_initialized():
        dist.init_process_group(backend=backend)
    return dist.get_rank(), dist.get_world_size()


def shard_range(n, rank, world):
    """Columns [lo, hi) of a batch of n that rank `rank` owns (contiguous, near-equal)."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def bucket_bounds(offsets):
    """[(start, stop)] per layer of a flat [W1,b1,W2,b2,...] buffer, in backward order."""
    return [(int(offsets[i]), int(offsets[i + 1])) for i in reversed(range(len(offsets) - 1))]


def allreduce_bucket(flat_g, bounds, group=None, async_op=True):
    """Sum one gradient bucket over the ranks in place; returns the work handle."""
    a, b = bounds
    return dist.all_reduce(flat_g[a:b], op=dist.ReduceOp.SUM, group=group, async_op=async_op)


def gradient_scale(world):
    """Factor applied to the summed gradient: the mean over ranks of per-rank mean losses."""
    return 1.0 / world


def reduce_loss(total, count, group=None):
    """Global (sum, count) of the per-rank nll totals for reporting."""
    t = torch.stack([total.reshape(()).to(torch.float64), count.reshape(()).to(torch.float64)])
    dist.all_reduce(t, group=group)
    return float(t[0]), int(t[1])
