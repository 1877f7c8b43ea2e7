"""Two ranks on two GPUs over NCCL (skipped with fewer than two devices): every rank draws the same seed-42
batch, keeps its rows, runs RWKV-5 forward+backward and the one collective of this library (parameter
gradients reduced over the local batch in fp32, all-reduced once).  Per-token outputs must equal the rows of
the single-GPU run bit for bit; the all-reduced gw / gu must equal the single-GPU sums to fp32 tolerance."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(dev, B, T, H, N):
    g = torch.Generator(device=dev)
    g.manual_seed(42)
    C, bf = H * N, torch.bfloat16
    full = lambda sc=1.0: torch.randn(B, T, C, generator=g, device=dev) * sc
    r, k, v = (full(0.5).to(bf) for _ in range(3))
    gy = full().to(bf)
    wraw = (torch.rand(H, N, generator=g, device=dev) * 5 - 6).to(bf)
    u = (torch.rand(H, N, generator=g, device=dev) * 2 - 1).to(bf)
    return r, k, v, gy, wraw, u


def _run(R, dev, r, k, v, gy, wraw, u, H):
    B, T, C = r.shape
    bf = torch.bfloat16
    ew = -torch.exp(wraw.float())
    eew = torch.exp(ew)
    y, gr, gk, gv = (torch.empty(B, T, C, dtype=bf, device=dev) for _ in range(4))
    gw, gu = torch.empty(B, C, dtype=bf, device=dev), torch.empty(B, C, dtype=bf, device=dev)
    R.ops.wkv5_forward(B, T, C, H, r, k, v, eew, u, y)
    R.ops.wkv5_backward(B, T, C, H, r, k, v, eew, ew, u, gy, gr, gk, gv, gw, gu)
    red = R.dist.ParamGradReducer(dev, 2 * C)
    red.add(gw); red.add(gu)
    red.launch()
    out = dict(y=y, gr=gr, gk=gk, gv=gv, gw=red.result(0).clone(), gu=red.result(1).clone())
    torch.cuda.synchronize(dev)
    return out


def _worker(rank, world, port, q):
    import torch.distributed as dist
    import rwkv_cuda_b200 as R
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, T, H, N = 4, 256, 4, 64
        r, k, v, gy, wraw, u = _inputs(dev, B, T, H, N)
        bl = B // world
        sl = slice(rank * bl, (rank + 1) * bl)
        part = _run(R, dev, r[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), gy[sl].contiguous(), wraw, u, H)
        dist.barrier()
        q.put((rank, {n: x.cpu() for n, x in part.items()}))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_reproduce_one_gpu():
    import torch.multiprocessing as mp
    import rwkv_cuda_b200 as R
    world, port = 2, 29731 + os.getpid() % 500
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(rk, world, port, q)) for rk in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    dev = torch.device("cuda", 0)
    B, T, H, N = 4, 256, 4, 64
    r, k, v, gy, wraw, u = _inputs(dev, B, T, H, N)
    whole = _run(R, dev, r, k, v, gy, wraw, u, H)   # no process group here: the local sum over the whole batch
    bl = B // world
    for rk in range(world):
        for n in ("y", "gr", "gk", "gv"):
            assert torch.equal(res[rk][n], whole[n][rk * bl:(rk + 1) * bl].cpu()), f"rank {rk}: {n}"
        for n in ("gw", "gu"):
            a, b = res[rk][n].double(), whole[n].cpu().double()
            assert (a - b).abs().max() <= 1e-5 * b.abs().max() + 1e-6, f"rank {rk}: {n}"
