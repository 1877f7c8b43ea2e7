"""GPU: the forward split over time (two-level scan) for RWKV-5 and RWKV-6 with state, against the fp64
oracle and against the unsplit forward; the reference's counterpart is the forward-only
wkv5_bf16/cuda/wkv5_cuda_v3.cu (static decay, no state)."""
import pytest
import torch

from oracle import wkv_oracle as O
from tests import helpers as Hh

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


@pytest.fixture(scope="module")
def R():
    import rwkv_cuda_b200 as R
    return R


def _v6_inputs(B, T, H, N, seed, shift=-3.0):
    g = Hh.gen(seed)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u = Hh.randn(g, B, T, C) + shift, Hh.rand(g, H, N, lo=-1, hi=1)
    s0 = 0.1 * Hh.randn(g, B, H, N, N)
    return r, k, v, w_raw, u, s0


@pytest.mark.parametrize("B,T,H,K", [(1, 1024, 2, 4), (2, 512, 3, 2), (1, 256, 1, 8), (1, 96, 2, 3)])
def test_rwkv6_state_forward_split_over_time(R, B, T, H, K):
    N = 64
    C = H * N
    r, k, v, w_raw, u, s0 = _v6_inputs(B, T, H, N, seed=11)
    xs = [x.to(BF).double() for x in (r, k, v, w_raw, u)]
    yo, sTo = O.wkv6(*xs, H, s0=s0.double(), return_state=True)
    rd, kd, vd, wd, ud = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, w_raw, u))
    s0d = s0.to(DEV)
    y, sT = torch.full((B, T, C), float("nan"), dtype=BF, device=DEV), torch.full((B, H, N, N), float("nan"), device=DEV)
    R.ops.wkv6state_forward_tsplit(B, T, C, H, rd, kd, vd, wd, ud, s0d, y, sT, segments=K)
    y1, sT1 = torch.empty_like(y), torch.empty_like(sT)
    R.ops.wkv6state_forward_ex(B, T, C, H, rd, kd, vd, wd, ud, s0d, y1, sT1)
    torch.cuda.synchronize()
    Hh.assert_close(y, yo, Hh.TOL_BF16, "y (split) against the oracle")
    Hh.assert_close(sT, sTo, Hh.TOL_BF16, "sT (split) against the oracle")
    # against the unsplit kernel: the same products inside a segment, start states combined in another order
    Hh.assert_close(y, y1.double().cpu(), Hh.TOL_BF16, "y split against unsplit")
    Hh.assert_close(sT, sT1.double().cpu(), Hh.TOL_BF16,
                    "sT split against unsplit")


def test_rwkv6_split_without_a_state(R):
    B, T, H, N, K = 1, 512, 2, 64, 4
    C = H * N
    r, k, v, w_raw, u, _ = _v6_inputs(B, T, H, N, seed=12)
    xs = [x.to(BF).double() for x in (r, k, v, w_raw, u)]
    yo = O.wkv6(*xs, H)
    rd, kd, vd, wd, ud = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, w_raw, u))
    y = torch.full((B, T, C), float("nan"), dtype=BF, device=DEV)
    R.ops.wkv6state_forward_tsplit(B, T, C, H, rd, kd, vd, wd, ud, None, y, None, segments=K)
    torch.cuda.synchronize()
    Hh.assert_close(y, yo, Hh.TOL_BF16, "y (split, zero start state)")


@pytest.mark.parametrize("B,T,H,K", [(1, 1024, 2, 4), (2, 256, 3, 2)])
def test_rwkv5_forward_split_over_time(R, B, T, H, K):
    N = 64
    C = H * N
    g = Hh.gen(21)
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u = Hh.rand(g, H, N, lo=-6, hi=-1), Hh.rand(g, H, N, lo=-1, hi=1)
    xs = [x.to(BF).double() for x in (r, k, v, w_raw, u)]
    yo = O.wkv5(*xs, H)
    rd, kd, vd, ud = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, u))
    eew = torch.exp(-torch.exp(w_raw.to(BF).float())).to(DEV).contiguous()
    y = torch.full((B, T, C), float("nan"), dtype=BF, device=DEV)
    R.ops.wkv5_forward_tsplit(B, T, C, H, rd, kd, vd, eew, ud, y, segments=K)
    y1 = torch.empty_like(y)
    R.ops.wkv5_forward(B, T, C, H, rd, kd, vd, eew, ud, y1)
    torch.cuda.synchronize()
    Hh.assert_close(y, yo, Hh.TOL_BF16, "y (split) against the oracle")
    Hh.assert_close(y, y1.double().cpu(), Hh.TOL_BF16, "y split against unsplit")


def test_split_with_a_decay_too_strong_for_the_chunked_form(R):
    """Log-decays below -5 per token: the chunked kernels raise their flag and the general-shape kernel redoes
    the whole call, split or not."""
    B, T, H, N, K = 1, 128, 2, 64, 2
    C = H * N
    r, k, v, w_raw, u, s0 = _v6_inputs(B, T, H, N, seed=13, shift=2.0)
    xs = [x.to(BF).double() for x in (r, k, v, w_raw, u)]
    yo, sTo = O.wkv6(*xs, H, s0=s0.double(), return_state=True)
    rd, kd, vd, wd, ud = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, w_raw, u))
    y, sT = torch.full((B, T, C), float("nan"), dtype=BF, device=DEV), torch.full((B, H, N, N), float("nan"), device=DEV)
    R.ops.wkv6state_forward_tsplit(B, T, C, H, rd, kd, vd, wd, ud, s0.to(DEV), y, sT, segments=K)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and torch.isfinite(sT).all()
    Hh.assert_close(y, yo, Hh.TOL_BF16, "y (split, strong decay)")
    Hh.assert_close(sT, sTo, Hh.TOL_BF16, "sT (split, strong decay)")


def test_split_rejects_segments_that_are_not_whole_chunks(R):
    B, T, H, N = 1, 96, 1, 64
    C = H * N
    z = torch.zeros(B, T, C, dtype=BF, device=DEV)
    u = torch.zeros(H, N, dtype=BF, device=DEV)
    with pytest.raises(Exception):
        R.ops.wkv6state_forward_tsplit(B, T, C, H, z, z, z, z, u, None, torch.empty_like(z), None, segments=4)   # 24 tokens


def test_split_pays_for_a_single_sequence_of_few_heads(R):
    """One long sequence of 8 heads on 148 SMs: the split forward is faster than the unsplit one (measured 2x at
    T = 16384 with the 16 segments that are chosen automatically); with 64 heads the automatic choice is not to
    split.  Prints the times."""
    dev = torch.device(DEV)
    assert R.ops.tsplit_segments(1, 4096, 64, dev) == 1
    B, T, H, N = 1, 16384, 8, 64
    C = H * N
    g = torch.Generator(device=DEV)
    g.manual_seed(5)
    mk = lambda sc=0.5: (sc * torch.randn(B, T, C, generator=g, device=DEV)).to(BF)
    r, k, v = mk(), mk(), mk()
    w = (torch.randn(B, T, C, generator=g, device=DEV) - 3.0).to(BF)
    u = (torch.rand(H, N, generator=g, device=DEV) * 2 - 1).to(BF)
    s0 = 0.1 * torch.randn(B, H, N, N, generator=g, device=DEV)
    y, sT = torch.empty(B, T, C, dtype=BF, device=DEV), torch.empty_like(s0)
    K = R.ops.tsplit_segments(B, T, H, dev)
    assert K >= 8

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 10

    t_plain = timed(lambda: R.ops.wkv6state_forward_ex(B, T, C, H, r, k, v, w, u, s0, y, sT))
    t_split = timed(lambda: R.ops.wkv6state_forward_tsplit(B, T, C, H, r, k, v, w, u, s0, y, sT))
    print(f"RWKV-6 forward B1 T16384 H8: unsplit {t_plain:.3f} ms, split into {K} segments (automatic) {t_split:.3f} ms")
    assert t_split < 0.8 * t_plain


@pytest.mark.parametrize("B,T,H", [(2, 256, 3), (1, 48, 2), (1, 2048, 1)])
def test_rwkv6_forward_kernels_agree(R, B, T, H):
    """The tcgen05 forward (32-token chunks) and the mma.sync forward (16-token chunks) of RWKV-6 with state:
    both against the oracle, and close to each other; the times of the benchmark shape are printed."""
    from rwkv_cuda_b200 import _lib
    N = 64
    C = H * N
    r, k, v, w_raw, u, s0 = _v6_inputs(B, T, H, N, seed=31)
    xs = [x.to(BF).double() for x in (r, k, v, w_raw, u)]
    yo, sTo = O.wkv6(*xs, H, s0=s0.double(), return_state=True)
    rd, kd, vd, wd, ud = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, w_raw, u))
    outs = {}
    try:
        for kern in (0, 1):
            _lib.call("rwkvb200_wkv6_select_forward", kern)
            y, sT = torch.full((B, T, C), float("nan"), dtype=BF, device=DEV), torch.full((B, H, N, N), float("nan"), device=DEV)
            R.ops.wkv6state_forward_ex(B, T, C, H, rd, kd, vd, wd, ud, s0.to(DEV), y, sT)
            torch.cuda.synchronize()
            assert _lib.lib().rwkvb200_device_status() == 0
            Hh.assert_close(y, yo, Hh.TOL_BF16, f"y, forward kernel {kern}")
            Hh.assert_close(sT, sTo, Hh.TOL_BF16, f"sT, forward kernel {kern}")
            outs[kern] = (y, sT)
    finally:
        _lib.call("rwkvb200_wkv6_select_forward", 1)
    Hh.assert_close(outs[1][0], outs[0][0].double().cpu(), Hh.TOL_BF16, "y, tcgen05 against mma.sync")


def test_rwkv6_forward_kernel_times(R):
    from rwkv_cuda_b200 import _lib
    B, T, H, N = 16, 4096, 64, 64
    C = H * N
    g = torch.Generator(device=DEV)
    g.manual_seed(5)
    mk = lambda sc=0.5: (sc * torch.randn(B, T, C, generator=g, device=DEV)).to(BF)
    r, k, v = mk(), mk(), mk()
    w = (torch.randn(B, T, C, generator=g, device=DEV) - 3.0).to(BF)
    u = (torch.rand(H, N, generator=g, device=DEV) * 2 - 1).to(BF)
    s0 = 0.1 * torch.randn(B, H, N, N, generator=g, device=DEV)
    y, sT = torch.empty(B, T, C, dtype=BF, device=DEV), torch.empty_like(s0)
    times = {}
    try:
        for kern in (0, 1):
            _lib.call("rwkvb200_wkv6_select_forward", kern)
            for _ in range(3):
                R.ops.wkv6state_forward_ex(B, T, C, H, r, k, v, w, u, s0, y, sT)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                R.ops.wkv6state_forward_ex(B, T, C, H, r, k, v, w, u, s0, y, sT)
            e1.record()
            torch.cuda.synchronize()
            times[kern] = e0.elapsed_time(e1) / 10
    finally:
        _lib.call("rwkvb200_wkv6_select_forward", 1)
    print(f"RWKV-6 forward B16 T4096 H64: mma.sync {times[0]:.3f} ms, tcgen05 {times[1]:.3f} ms")
    assert _lib.lib().rwkvb200_device_status() == 0


@pytest.mark.parametrize("B,T,H", [(2, 256, 3), (1, 48, 2), (1, 1024, 1)])
def test_rwkv6_backward_kernels_agree(R, B, T, H):
    """The tcgen05 backward (32-token chunks) and the mma.sync backward (16-token chunks) of RWKV-6 with state and a
    gradient of the final state: both against autograd through the fp64 oracle, and close to each other."""
    from rwkv_cuda_b200 import _lib
    N = 64
    C = H * N
    r, k, v, w_raw, u, s0 = _v6_inputs(B, T, H, N, seed=37)
    g = Hh.gen(38)
    gy, dsT = Hh.randn(g, B, T, C), Hh.randn(g, B, H, N, N)
    xs = [x.to(BF).double().requires_grad_(True) for x in (r, k, v, w_raw, u)] + [s0.double().requires_grad_(True)]
    yo, sTo = O.wkv6(*xs[:5], H, s0=xs[5], return_state=True)
    torch.autograd.backward([yo, sTo], [gy.to(BF).double(), dsT.double()])
    rd, kd, vd, wd, ud, gd = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, w_raw, u, gy))
    s0d, dsTd = s0.to(DEV), dsT.to(DEV)
    names = ("gr", "gk", "gv", "gw", "gu", "ds0")
    outs = {}
    try:
        for kern in (0, 1):
            _lib.call("rwkvb200_wkv6_select_forward", kern)
            nan = float("nan")
            gr, gk, gv, gw = (torch.full((B, T, C), nan, dtype=BF, device=DEV) for _ in range(4))
            gu, ds0 = torch.full((B, C), nan, dtype=BF, device=DEV), torch.full((B, H, N, N), nan, device=DEV)
            R.ops.wkv6state_backward_ex(B, T, C, H, rd, kd, vd, wd, ud, s0d, gd, dsTd, gr, gk, gv, gw, gu, ds0)
            torch.cuda.synchronize()
            assert _lib.lib().rwkvb200_device_status() == 0
            got = (gr, gk, gv, gw, gu.float().sum(0), ds0)
            for x, want, name in zip(got, [xx.grad for xx in xs], names):
                Hh.assert_close(x, want, Hh.TOL_BF16, f"{name}, backward kernel {kern}")
            outs[kern] = got
    finally:
        _lib.call("rwkvb200_wkv6_select_forward", 1)
    for a, b, name in zip(outs[1], outs[0], names):
        Hh.assert_close(a, b.double().cpu(), Hh.TOL_BF16, f"{name}, tcgen05 against mma.sync")


@pytest.mark.parametrize("B,T,H,shift", [(2, 256, 3, -3.0), (1, 48, 2, -3.0), (2, 128, 2, 2.0)])
def test_rwkv6_saved_states_flow(R, B, T, H, shift):
    """Forward that keeps the chunk-start states + backward that uses them (also with decays too strong for the
    chunked form: flagged units are redone by the general-shape kernels in both passes), against the oracle."""
    N = 64
    C = H * N
    r, k, v, w_raw, u, s0 = _v6_inputs(B, T, H, N, seed=41, shift=shift)
    g = Hh.gen(42)
    gy, dsT = Hh.randn(g, B, T, C), Hh.randn(g, B, H, N, N)
    xs = [x.to(BF).double().requires_grad_(True) for x in (r, k, v, w_raw, u)] + [s0.double().requires_grad_(True)]
    yo, sTo = O.wkv6(*xs[:5], H, s0=xs[5], return_state=True)
    torch.autograd.backward([yo, sTo], [gy.to(BF).double(), dsT.double()])
    rd, kd, vd, wd, ud, gd = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, w_raw, u, gy))
    s0d, dsTd = s0.to(DEV), dsT.to(DEV)
    nan = float("nan")
    y, sT = torch.full((B, T, C), nan, dtype=BF, device=DEV), torch.full((B, H, N, N), nan, device=DEV)
    saved = torch.empty(R.ops.wkv6_saved_bytes(B, T, C), dtype=torch.uint8, device=DEV)
    valid = R.ops.wkv6state_forward_saved(B, T, C, H, rd, kd, vd, wd, ud, s0d, y, sT, saved)
    assert valid
    # another call on the same stream in between must not disturb the saved flags
    R.ops.wkv6state_forward_ex(B, T, C, H, rd, kd, vd, (wd.float() - 6.0).to(BF), ud, s0d, torch.empty_like(y), torch.empty_like(sT))
    gr, gk, gv, gw = (torch.full((B, T, C), nan, dtype=BF, device=DEV) for _ in range(4))
    gu, ds0 = torch.full((B, C), nan, dtype=BF, device=DEV), torch.full((B, H, N, N), nan, device=DEV)
    R.ops.wkv6state_backward_saved(B, T, C, H, rd, kd, vd, wd, ud, s0d, gd, dsTd, gr, gk, gv, gw, gu, ds0, saved, valid)
    torch.cuda.synchronize()
    Hh.assert_close(y, yo.detach(), Hh.TOL_BF16, "y")
    Hh.assert_close(sT, sTo.detach(), Hh.TOL_BF16, "sT")
    for x, want, name in zip((gr, gk, gv, gw, gu.float().sum(0), ds0), [xx.grad for xx in xs], ("gr", "gk", "gv", "gw", "gu", "ds0")):
        assert torch.isfinite(x.float()).all(), name
        if name == "gw" and shift > 0:
            continue   # e^2 and more per token: the decay gradient is below what bf16 inputs resolve
        Hh.assert_close(x, want, Hh.TOL_BF16, f"{name} (saved-states flow)")


@pytest.mark.parametrize("B,T,H,hi", [(2, 256, 3, -1.0), (1, 48, 2, -1.0), (2, 64, 2, 2.5)])
def test_rwkv5_saved_states_flow(R, B, T, H, hi):
    """RWKV-5: forward that keeps the chunk-start states + backward that uses them, with the fp32 partials of the
    parameter gradients, against the oracle (hi = 2.5: decays too strong for the chunked form in some channels)."""
    N = 64
    C = H * N
    g = Hh.gen(51)
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.rand(g, H, N, lo=-6 if hi < 0 else -1, hi=hi), Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    xs = [x.to(BF).double().requires_grad_(True) for x in (r, k, v, w_raw, u)]
    yo = O.wkv5(*xs, H)
    yo.backward(gy.to(BF).double())
    rd, kd, vd, ud, gd = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, u, gy))
    ew = -torch.exp(w_raw.to(BF).float()).to(DEV).contiguous()
    eew = torch.exp(ew).contiguous()
    nan = float("nan")
    y = torch.full((B, T, C), nan, dtype=BF, device=DEV)
    saved = torch.empty(R.ops.wkv5_saved_bytes(B, T, C), dtype=torch.uint8, device=DEV)
    valid = R.ops.wkv5_forward_saved(B, T, C, H, rd, kd, vd, eew, ud, y, saved)
    assert valid
    gr, gk, gv = (torch.full((B, T, C), nan, dtype=BF, device=DEV) for _ in range(3))
    gw, gu = torch.full((B, C), nan, dtype=BF, device=DEV), torch.full((B, C), nan, dtype=BF, device=DEV)
    gw32, gu32 = torch.full((B, C), nan, device=DEV), torch.full((B, C), nan, device=DEV)
    R.ops.wkv5_backward_saved(B, T, C, H, rd, kd, vd, eew, ew, ud, gd, gr, gk, gv, gw, gu, saved, valid, gw32, gu32)
    torch.cuda.synchronize()
    got = (y, gr, gk, gv, gw32.sum(0), gu32.sum(0))
    for x, want, name in zip(got, [yo.detach()] + [xx.grad for xx in xs], ("y", "gr", "gk", "gv", "gw", "gu")):
        assert torch.isfinite(x.float()).all(), name
        Hh.assert_close(x, want, Hh.TOL_BF16, f"{name} (RWKV-5 saved-states flow)")
    Hh.assert_close(gw.float().sum(0), xs[3].grad, Hh.TOL_BF16, "gw from the bf16 partials")


@pytest.mark.parametrize("B,T,H", [(2, 256, 3), (1, 48, 2)])
def test_rwkv6_backward_without_tensor_maps(R, B, T, H):
    """The tcgen05 RWKV-6 backward when it cannot make tensor maps (test hook): it loads its inputs with plain loads
    instead of TMA and the gradients are bit-identical.  The states come from a forward that ran with maps."""
    from rwkv_cuda_b200 import _lib
    N = 64
    C = H * N
    r, k, v, w_raw, u, s0 = _v6_inputs(B, T, H, N, seed=51)
    g = Hh.gen(52)
    gy, dsT = Hh.randn(g, B, T, C), Hh.randn(g, B, H, N, N)
    rd, kd, vd, wd, ud, gd = (x.to(BF).to(DEV).contiguous() for x in (r, k, v, w_raw, u, gy))
    s0d, dsTd = s0.to(DEV), dsT.to(DEV)
    y, sT = torch.empty(B, T, C, dtype=BF, device=DEV), torch.empty(B, H, N, N, device=DEV)
    saved = torch.empty(R.ops.wkv6_saved_bytes(B, T, C), dtype=torch.uint8, device=DEV)
    valid = R.ops.wkv6state_forward_saved(B, T, C, H, rd, kd, vd, wd, ud, s0d, y, sT, saved)
    assert valid

    def run():
        nan = float("nan")
        gr, gk, gv, gw = (torch.full((B, T, C), nan, dtype=BF, device=DEV) for _ in range(4))
        gu, ds0 = torch.full((B, C), nan, dtype=BF, device=DEV), torch.full((B, H, N, N), nan, device=DEV)
        R.ops.wkv6state_backward_saved(B, T, C, H, rd, kd, vd, wd, ud, s0d, gd, dsTd, gr, gk, gv, gw, gu, ds0, saved, valid)
        torch.cuda.synchronize()
        return gr, gk, gv, gw, gu, ds0

    a = run()
    try:
        _lib.call("rwkvb200_test_disable_tensor_maps", 1)
        b = run()
    finally:
        _lib.call("rwkvb200_test_disable_tensor_maps", 0)
    assert _lib.lib().rwkvb200_device_status() == 0
    for x, y2, name in zip(a, b, ("gr", "gk", "gv", "gw", "gu", "ds0")):
        assert torch.isfinite(x.float()).all(), name
        assert torch.equal(x, y2), name
