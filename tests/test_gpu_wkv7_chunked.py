"""The tensor-core (chunked) RWKV-7 kernels, forced on, against the fp64 oracle."""
import pytest
import torch

from oracle import wkv_oracle as O
from tests import helpers as Hh

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=[2, 3, 4, 5], ids=["mma_sync", "tcgen05_fwd", "tcgen05_fwd_bwd", "producer_consumer"])
def R(request):
    """2 = mma.sync chunked kernels, 3 = tcgen05 forward with the same backward."""
    import rwkv_cuda_b200 as R
    from rwkv_cuda_b200 import _lib
    _lib.call("rwkvb200_wkv7_select_path", request.param)
    yield R
    _lib.call("rwkvb200_wkv7_select_path", 0)
    assert _lib.lib().rwkvb200_device_status() == 0, "a bounded wait expired inside a tcgen05 kernel"


@pytest.mark.parametrize("B,T,H", [(1, 16, 1), (2, 64, 2), (1, 512, 3)])
@pytest.mark.parametrize("use_s0", [True, False])
def test_forward(R, B, T, H, use_s0):
    N = 64
    bf = torch.bfloat16
    inp = Hh.v7_inputs(B, T, H, N, seed=5)
    inp64 = {n: (x.to(bf).double() if n not in ("s0", "dsT") else x.double()) for n, x in inp.items()}
    y64, sT64 = O.wkv7(*(inp64[n] for n in ("r", "w", "k", "v", "a", "b")), H, s0=inp64["s0"] if use_s0 else None)
    d = {n: inp[n].to(bf).to(DEV).view(B, T, H, N).contiguous() for n in ("r", "w", "k", "v", "a", "b")}
    s0 = inp["s0"].to(DEV) if use_s0 else None
    y = torch.full((B, T, H, N), float("nan"), dtype=bf, device=DEV)
    sT = torch.full((B, H, N, N), float("nan"), device=DEV)
    s = torch.full((B, H, T // 16, N, N), float("nan"), device=DEV)
    sa = torch.full((B, T, H, N), float("nan"), device=DEV)
    R.ops.wkv7_forward(s0, d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], y, sT, s, sa)
    torch.cuda.synchronize()
    print("y", Hh.assert_close(y, y64, Hh.TOL_BF16, "y"))
    print("sT", Hh.assert_close(sT, sT64, Hh.TOL_BF16, "sT"))
    assert torch.isfinite(s).all() and torch.isfinite(sa).all()
    # saved state of chunk 0 is the initial state
    want0 = inp["s0"] if use_s0 else torch.zeros(B, H, N, N)
    assert torch.equal(s[:, :, 0].cpu(), want0)


def _run_both(R, inp, H, use_s0, use_sT):
    B, T, C = inp["r"].shape
    N = C // H
    bf = torch.bfloat16
    d = {n: inp[n].to(bf).to(DEV).view(B, T, H, N).contiguous() for n in ("r", "w", "k", "v", "a", "b", "dy")}
    s0 = inp["s0"].to(DEV) if use_s0 else None
    dsT = inp["dsT"].to(DEV) if use_sT else None
    nan = float("nan")
    y = torch.full((B, T, H, N), nan, dtype=bf, device=DEV)
    sT = torch.full((B, H, N, N), nan, device=DEV) if use_sT else None
    s = torch.full((B, H, T // 16, N, N), nan, device=DEV)
    sa = torch.full((B, T, H, N), nan, device=DEV)
    R.ops.wkv7_forward(s0, d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], y, sT, s, sa)
    g = [torch.full((B, T, H, N), nan, dtype=bf, device=DEV) for _ in range(6)]
    ds0 = torch.full((B, H, N, N), nan, device=DEV) if use_s0 else None
    R.ops.wkv7_backward(d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], d["dy"], dsT, s, sa, ds0, *g)
    torch.cuda.synchronize()
    return dict(y=y, sT=sT, ds0=ds0, **dict(zip(("dr", "dw", "dk", "dv", "da", "db"), g)))


@pytest.mark.parametrize("B,T,H", [(1, 16, 1), (2, 64, 2), (1, 512, 3), (1, 2048, 1)])
@pytest.mark.parametrize("use_s0,use_sT", [(True, True), (False, False), (True, False)])
def test_forward_backward(R, B, T, H, use_s0, use_sT):
    N = 64
    bf = torch.bfloat16
    inp = Hh.v7_inputs(B, T, H, N, seed=7)
    inp64 = {n: (x.to(bf).double() if n not in ("s0", "dsT") else x.double()) for n, x in inp.items()}
    want = Hh.v7_oracle(inp64, H, use_s0=use_s0, use_dsT=use_sT)
    out = _run_both(R, inp, H, use_s0, use_sT)
    names = ["y", "dr", "dw", "dk", "dv", "da", "db"] + (["ds0"] if use_s0 else []) + (["sT"] if use_sT else [])
    rep = {n: "%.2e" % Hh.assert_close(out[n], want[n], Hh.TOL_BF16, n)[1] for n in names}
    print(rep)


def _set_path(p):
    from rwkv_cuda_b200 import _lib
    _lib.call("rwkvb200_wkv7_select_path", p)


@pytest.mark.parametrize("B,T,H", [(1, 64, 3), (3, 32, 64), (5, 32, 64)])
def test_kernel_choice_by_grid_size_is_bit_exact(B, T, H):
    """The producer/consumer kernels (small grids) and the plain ones (B*H above the SM count) do the
    same arithmetic in the same order: forced either way, and chosen automatically on both sides of
    the threshold, they must agree bit for bit."""
    import rwkv_cuda_b200 as R
    inp = Hh.v7_inputs(B, T, H, 64, seed=11)
    outs = {}
    try:
        for p in (3, 5, 0):
            _set_path(p)
            outs[p] = _run_both(R, inp, H, True, True)
    finally:
        _set_path(0)
    for n in ("y", "sT", "dr", "dw", "dk", "dv", "da", "db", "ds0"):
        assert torch.equal(outs[3][n], outs[5][n]), n
        assert torch.equal(outs[3][n], outs[0][n]), n
