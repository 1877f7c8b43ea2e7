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


class ParamGradReducer:
    """Parameter gradients of one backward call, summed over the local batch and over the ranks.

    `add(partial)` reduces a per-batch partial (B, n) -- what the backward kernels emit -- over the batch
    in fp32 into the next slice of ONE fp32 buffer (no bf16 round trip), on the caller's stream;
    `launch()` enqueues the all-reduce of that buffer on a side stream as soon as the reductions are
    done, so it overlaps whatever the caller enqueues next; `result(i)` waits for it and returns the
    i-th reduced gradient as a view of the buffer.  Without a process group it is the local sum."""

    def __init__(self, device, capacity, group=None):
        self.buf = torch.zeros(capacity, dtype=torch.float32, device=device)
        self.side = torch.cuda.Stream(device)
        self.group, self.spans, self.off, self.work, self.done = group, [], 0, None, None

    def add(self, partial):
        from . import ops
        n = partial.numel() // partial.shape[0]
        if self.off + n > self.buf.numel():
            raise ValueError("ParamGradReducer: capacity exceeded")
        ops.reduce_batch_partials(partial, self.buf[self.off:self.off + n])
        self.spans.append((self.off, n))
        self.off += n
        return len(self.spans) - 1

    def launch(self):
        cur = torch.cuda.current_stream(self.buf.device)
        self.side.wait_stream(cur)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            with torch.cuda.stream(self.side):
                self.work = dist.all_reduce(self.buf[:self.off], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self.done = self.side.record_event() if self.work is None else None

    def result(self, i):
        cur = torch.cuda.current_stream(self.buf.device)
        if self.work is not None:
            self.work.wait()          # makes the current stream wait for the collective
            self.work = None
        elif self.done is not None:
            cur.wait_event(self.done)
        lo, n = self.spans[i]
        return self.buf[lo:lo + n]

    def reset(self):
        self.spans, self.off, self.work, self.done = [], 0, None, None
