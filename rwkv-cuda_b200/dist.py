"""Multi-GPU plumbing: one process per GPU, the batch is sharded, nothing else is exchanged.

Every operator here is independent across batch rows, so each rank runs the kernels on its
own slice of dim 0 and no data-path collective exists.  The only cross-rank step is the sum
of the parameter gradients (gw/gu of RWKV-4/5/5a/6, the conv filter gradient, ds0 in
state-tuning use), which are tiny: they are packed into ONE fp32 buffer and all-reduced once.
"""
import torch
import torch.distributed as dist


def shard_bounds(n, world_size, rank):
    """[lo, hi) of the contiguous batch slice of `rank`; the first n % world_size ranks get one more row."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} / world_size {world_size}")
    base, rem = divmod(n, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(t, world_size=None, rank=None, dim=0):
    """This rank's slice of `t` along the batch dimension (a contiguous copy)."""
    world_size = dist.get_world_size() if world_size is None else world_size
    rank = dist.get_rank() if rank is None else rank
    lo, hi = shard_bounds(t.shape[dim], world_size, rank)
    return t.narrow(dim, lo, hi - lo).contiguous()


def allreduce_param_grads(grads, group=None, async_op=False):
    """Sum a list of small parameter-gradient tensors over all ranks with ONE all-reduce.

    The tensors are flattened into one fp32 buffer (so bf16 partials are summed in fp32, not
    rounded per rank), reduced, and written back in place.  With async_op=True returns a
    callable that waits for the collective and then scatters the result back.
    """
    grads = [g for g in grads if g is not None]
    if not grads:
        return (lambda: None) if async_op else None
    flat = torch.cat([g.detach().reshape(-1).float() for g in grads])
    work = None
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)

    def finish():
        if work is not None and async_op:
            work.wait()
        off = 0
        for g in grads:
            n = g.numel()
            g.detach().copy_(flat[off:off + n].view_as(g).to(g.dtype))
            off += n

    if async_op:
        return finish
    finish()
    return None
