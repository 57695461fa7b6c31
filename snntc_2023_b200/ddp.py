"""Data-parallel plumbing of an SNN-TC train step: batch sharding and the one collective of the step.

Samples are independent in the forward and in dX; dW is a sum over samples. So the batch is split
evenly over the ranks, weights are replicated, every rank's backward kernels write its dW into one
flat fp32 bucket (SnnNet.flat_grad), and the step needs exactly one all-reduce of that bucket.
The functions are backend-agnostic (NCCL on GPUs, gloo in the CPU tests).
"""
import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """[start, stop) of this rank's share of n samples; shares differ by at most one sample."""
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def bucket_layout(shapes):
    """Offsets of each weight tensor inside the flat bucket: [(offset, numel, shape)], total."""
    out, off = [], 0
    for s in shapes:
        n = 1
        for d in s:
            n *= int(d)
        out.append((off, n, tuple(int(d) for d in s)))
        off += n
    return out, off


def allreduce_mean_(flat, world=None, group=None):
    """In-place mean of the flat gradient bucket over all ranks (sum all-reduce, then 1/world).
    The loss of each rank is a mean over ITS shard, so the mean over ranks is the gradient of the
    mean over the global batch when shards are equal."""
    if not dist.is_available() or not dist.is_initialized():
        return flat
    world = world or dist.get_world_size(group)
    if world == 1:
        return flat
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    flat.mul_(1.0 / world)
    return flat


def broadcast_(flat, src=0, group=None):
    """Make every rank start from rank `src`'s parameters."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(flat, src=src, group=group)
    return flat
