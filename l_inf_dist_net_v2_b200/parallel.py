"""Data-parallel plumbing for the operator: the batch dimension shards with no communication; the only
exchange is the all-reduce (mean) of parameter gradients that follows the grad_weight kernels, as
DistributedDataParallel does in the reference (main.py:357), and the averaging of a few scalar metrics
(main.py:60-64).  Works with any torch.distributed backend (NCCL on GPUs, gloo in CPU tests)."""
import torch
import torch.distributed as dist

__all__ = ["shard_bounds", "shard_batch", "allreduce_mean_", "average_scalars"]


def shard_bounds(n, rank, world):
    """Rows [lo, hi) of a global batch of n that rank `rank` of `world` owns: equal contiguous shards of
    n // world rows (main.py:346-348); n must be divisible by world."""
    if n % world != 0:
        raise ValueError(f"global batch {n} is not divisible by world size {world}")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_batch(t, rank, world):
    lo, hi = shard_bounds(t.size(0), rank, world)
    return t[lo:hi]


def allreduce_mean_(tensors, group=None, bucket_bytes=64 << 20):
    """In-place mean over ranks of every tensor in `tensors`.  Tensors are packed into flat buckets of at
    most `bucket_bytes` (one collective per bucket; a tensor larger than a bucket travels alone, in place)."""
    world = dist.get_world_size(group)
    if world == 1:
        return
    # NCCL averages inside the collective; other backends (gloo) sum, then one division pass follows
    avg = dist.get_backend(group) == "nccl"
    bucket, size = [], 0

    def reduce_(t):
        if avg:
            dist.all_reduce(t, op=dist.ReduceOp.AVG, group=group)
        else:
            dist.all_reduce(t, group=group)
            t.div_(world)

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        if len(bucket) == 1 and bucket[0].is_contiguous():
            reduce_(bucket[0])
        else:
            flat = torch.cat([b.reshape(-1) for b in bucket])
            reduce_(flat)
            off = 0
            for b in bucket:
                b.copy_(flat[off:off + b.numel()].view_as(b))
                off += b.numel()
        bucket, size = [], 0

    for t in tensors:
        nbytes = t.numel() * t.element_size()
        if size + nbytes > bucket_bytes:
            flush()
        bucket.append(t)
        size += nbytes
    flush()


def average_scalars(*values, device=None, group=None):
    """Mean over ranks of a few python floats (assumes equal shard sizes, like the reference)."""
    t = torch.tensor(values, dtype=torch.float32, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, group=group)
        t /= dist.get_world_size(group)
    return t.tolist()
