"""The tensor-core (chunked) RWKV-7 kernels, forced on, against the fp64 oracle."""
import pytest
import torch

from oracle import wkv_oracle as O
from tests import helpers as Hh

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=[(2, 1), (2, 2), (0, 0)], ids=["one_group", "two_stage", "automatic"])
def R(request):
    """(kernel path, backward form): path 2 = tensor-core kernels or an error, 0 = automatic; backward form
    1 = one warp group per chunk, 2 = two groups on consecutive chunks, 0 = chosen by the size of the launch."""
    import rwkv_cuda_b200 as R
    from rwkv_cuda_b200 import _lib
    _lib.call("rwkvb200_wkv7_select_path", request.param[0])
    _lib.call("rwkvb200_wkv7_select_form", request.param[1])
    yield R
    _lib.call("rwkvb200_wkv7_select_path", 0)
    _lib.call("rwkvb200_wkv7_select_form", 0)
    assert _lib.lib().rwkvb200_device_status() == 0, "a bounded wait expired inside a tcgen05 kernel"


@pytest.mark.parametrize("B,T,H", [(1, 16, 1), (1, 32, 1), (1, 48, 2), (2, 64, 2), (1, 512, 3)])
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
    # saved: the state at the start of every 32-token chunk; chunk 0 holds the initial state
    assert torch.isfinite(s[:, :, : (T + 31) // 32]).all()
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


@pytest.mark.parametrize("B,T,H", [(1, 16, 1), (1, 48, 2), (2, 64, 2), (1, 512, 3), (1, 2048, 1)])
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


def _set_form(f):
    from rwkv_cuda_b200 import _lib
    _lib.call("rwkvb200_wkv7_select_form", f)


def _set_path(p):
    from rwkv_cuda_b200 import _lib
    _lib.call("rwkvb200_wkv7_select_path", p)


def test_results_do_not_depend_on_the_grid():
    """A (batch, head) unit is computed by one thread block on its own: its results are bit-identical
    whether it runs alone or among 320 units (more than one per SM, several per SM in flight)."""
    import rwkv_cuda_b200 as R
    _set_form(1)   # the automatic choice would take different backward kernels for the two launches
    H, T = 64, 64
    big = Hh.v7_inputs(5, T, H, 64, seed=11)
    out_big = _run_both(R, big, H, True, True)
    b, h = 3, 17
    one = {n: (x[b : b + 1, :, h * 64 : (h + 1) * 64] if x.dim() == 3 else x[b : b + 1, h : h + 1]).contiguous() for n, x in big.items()}
    out_one = _run_both(R, one, 1, True, True)
    for n in ("y", "dr", "dw", "dk", "dv", "da", "db"):
        assert torch.equal(out_big[n][b, :, h], out_one[n][0, :, 0]), n
    for n in ("sT", "ds0"):
        assert torch.equal(out_big[n][b, h], out_one[n][0, 0]), n
    _set_form(0)


def test_kernel_forms_agree():
    """The two-stage backward runs the same products as the one-group backward: everything but dw is
    bit-identical, dw agrees to one bf16 ulp (the compiler fuses its last multiply-adds differently)."""
    import rwkv_cuda_b200 as R
    inp = Hh.v7_inputs(2, 512, 3, 64, seed=13)
    outs = {}
    try:
        for form in (1, 2):
            _set_form(form)
            outs[form] = _run_both(R, inp, 3, True, True)
    finally:
        _set_form(0)
    for n in ("sT", "dr", "dk", "dv", "da", "db", "ds0"):
        assert torch.equal(outs[1][n], outs[2][n]), n
    assert O.err_ratio(outs[1]["y"].double().cpu(), outs[2]["y"].double().cpu()) < 1e-4
    a, b = outs[1]["dw"].float(), outs[2]["dw"].float()
    assert (a - b).abs().max() <= 2.0 ** -7 * a.abs().max()
    assert (a != b).float().mean() < 1e-3


def test_bounded_wait_runs_out_and_the_library_recovers():
    """With the test hook the first product of the next forward is not issued, so the wait for it runs
    out (nothing is in flight): the kernel records its status, releases tensor memory and returns; after
    a reset the next call is correct again."""
    import rwkv_cuda_b200 as R
    from rwkv_cuda_b200 import _lib
    L = _lib.lib()
    assert L.rwkvb200_device_status() == 0
    inp = Hh.v7_inputs(1, 64, 2, 64, seed=3)
    good = _run_both(R, inp, 2, True, True)
    _lib.call("rwkvb200_wkv7_test_expire_next_forward")
    bad = _run_both(R, inp, 2, True, True)
    assert L.rwkvb200_device_status() == 11
    # the units whose wait ran out are marked: their first y element and first sT element are NaN
    assert torch.isnan(bad["y"].float()).any() and torch.isnan(bad["sT"]).any()
    assert L.rwkvb200_device_status() == 11, "the status word is sticky"
    _lib.call("rwkvb200_device_status_clear")
    assert L.rwkvb200_device_status() == 0
    again = _run_both(R, inp, 2, True, True)
    for n in good:
        assert torch.equal(good[n], again[n]), n
    assert L.rwkvb200_device_status() == 0


@pytest.mark.parametrize("form", [1, 2])
@pytest.mark.parametrize("B,T,H", [(2, 64, 2), (1, 48, 2), (1, 512, 3), (1, 16400, 2)])
def test_paths_without_tensor_maps_agree(form, B, T, H):
    """With the test hook that makes every tensor map fail, the backward kernels load their inputs with plain loads
    (and the forward falls back to its one-group form): the gradients are bit-identical to those of the TMA paths,
    since only the way the same words reach the registers differs."""
    import rwkv_cuda_b200 as R
    from rwkv_cuda_b200 import _lib
    inp = Hh.v7_inputs(B, T, H, 64, seed=23)
    try:
        _set_path(2)
        _set_form(form)
        with_maps = _run_both(R, inp, H, True, True)
        _lib.call("rwkvb200_test_disable_tensor_maps", 1)
        without = _run_both(R, inp, H, True, True)
    finally:
        _lib.call("rwkvb200_test_disable_tensor_maps", 0)
        _set_form(0)
        _set_path(0)
    assert _lib.lib().rwkvb200_device_status() == 0
    for n in ("dr", "dw", "dk", "dv", "da", "db", "ds0"):
        assert torch.equal(with_maps[n], without[n]), n
    # the forward differs in form (staged with maps, one group without when form != 1): equal up to rounding
    for n in ("y", "sT"):
        assert (with_maps[n].float() - without[n].float()).abs().max() <= 2e-2 * with_maps[n].float().abs().max(), n
