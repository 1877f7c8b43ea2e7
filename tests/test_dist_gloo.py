"""CPU tier: the multi-GPU plumbing on world-size-2 gloo ranks (batch sharding, the packed
parameter-gradient all-reduce)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import rwkv_cuda_b200 as R
from oracle import wkv_oracle as O


def test_shard_bounds_cover_the_batch():
    for n in (1, 2, 7, 16):
        for ws in (1, 2, 3, 8):
            spans = [R.dist.shard_bounds(n, ws, r) for r in range(ws)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    with pytest.raises(ValueError):
        R.dist.shard_bounds(4, 2, 2)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                     # every rank builds the same full batch ...
        B, T, H, N = 4, 6, 2, 4
        r, k, v = (torch.randn(B, T, H * N, dtype=torch.float64) for _ in range(3))
        w, u = torch.randn(H, N, dtype=torch.float64) - 1, torch.randn(H, N, dtype=torch.float64)
        gy = torch.randn(B, T, H * N, dtype=torch.float64)
        # ... the full-batch answer (what one GPU would compute)
        wf, uf = w.clone().requires_grad_(True), u.clone().requires_grad_(True)
        O.wkv5(r, k, v, wf, uf, H).backward(gy)
        # ... and its own shard
        rs, ks, vs, gs = (R.dist.shard_batch(x) for x in (r, k, v, gy))
        wl, ul = w.clone().requires_grad_(True), u.clone().requires_grad_(True)
        ys = O.wkv5(rs, ks, vs, wl, ul, H)
        ys.backward(gs)
        lo, hi = R.dist.shard_bounds(B, world, rank)
        ok_y = torch.equal(ys.detach(), O.wkv5(r, k, v, w, u, H)[lo:hi])   # per-token outputs need no exchange
        gw, gu = wl.grad.clone().to(torch.bfloat16), ul.grad.clone()         # a bf16 partial, as the kernels emit
        wait = R.dist.allreduce_param_grads([gw, None, gu], async_op=True)
        wait()
        err_w = (gw.double() - wf.grad).abs().max().item() / wf.grad.abs().max().item()
        err_u = (gu - uf.grad).abs().max().item() / uf.grad.abs().max().item()
        q.put((rank, ok_y, err_w, err_u))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_result():
    world, port = 2, 29631 + os.getpid() % 500
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, ok_y, err_w, err_u in res:
        assert ok_y, f"rank {rank}: sharded outputs differ from the full-batch run"
        assert err_u < 1e-6           # packed and summed in fp32
        assert err_w < 1e-2          # summed in fp32, written back to the bf16 partial


def test_allreduce_is_identity_without_a_process_group():
    g = [torch.ones(3), torch.full((2, 2), 2.0, dtype=torch.bfloat16)]
    R.dist.allreduce_param_grads(g)
    assert torch.equal(g[0], torch.ones(3)) and torch.equal(g[1].float(), torch.full((2, 2), 2.0))
