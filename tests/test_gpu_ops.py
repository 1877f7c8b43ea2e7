"""GPU parity: every operator of the library, through the C ABI, against the fp64 oracle and
the golden vectors made from the reference formulas."""
import os

import numpy as np
import pytest
import torch

from oracle import wkv_oracle as O
from tests import helpers as Hh

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def R():
    import rwkv_cuda_b200 as R
    R._lib.lib()  # must load: there is no fallback
    return R


def golden(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: torch.from_numpy(np.asarray(z[k])) for k in z.files}


def sentinel(*shape, dtype=torch.float32):
    """Output buffers start filled with junk so that unwritten elements show up
    (the trick of wkv6_state/run.py:102)."""
    return torch.empty(*shape, dtype=torch.float32, device=DEV).uniform_(-100, 100).to(dtype)


# ------------------------------------------------------------------ RWKV-4
def run_wkv4(R, w_raw, u, k, v, gy):
    B, T, C = k.shape
    wd, ud, kd, vd, gd = (x.float().to(DEV).contiguous() for x in (-torch.exp(w_raw.double()), u, k, v, gy))
    y = sentinel(B, T, C)
    R.ops.wkv4_forward(B, T, C, wd, ud, kd, vd, y)
    gw = torch.zeros(B, C, device=DEV)
    gu = torch.zeros(B, C, device=DEV)
    gk, gv = sentinel(B, T, C), sentinel(B, T, C)
    R.ops.wkv4_backward(B, T, C, wd, ud, kd, vd, gd, gw, gu, gk, gv)
    return y, gw.sum(0), gu.sum(0), gk, gv


def test_wkv4_golden(R, golden_dir):
    g = golden(golden_dir, "wkv4")
    yy = g["y"].clone().requires_grad_(True)
    O.strange_loss(yy).backward()
    y, gw, gu, gk, gv = run_wkv4(R, g["w"], g["u"], g["k"], g["v"], yy.grad)
    for got, name in ((y, "y"), (gw, "gw"), (gu, "gu"), (gk, "gk"), (gv, "gv")):
        Hh.assert_close(got, g[name], Hh.TOL_FP32_STRICT, "wkv4 " + name)


@pytest.mark.parametrize("B,T,C", [(4, 256, 256), (2, 768, 96), (3, 37, 5), (1, 5000, 33)])
def test_wkv4_oracle(R, B, T, C):
    g = Hh.gen(42)
    w_raw = Hh.rand(g, C, lo=-4, hi=1)
    u = Hh.rand(g, C, lo=-1, hi=1)
    k, v, gy = 0.5 * Hh.randn(g, B, T, C), Hh.randn(g, B, T, C), Hh.randn(g, B, T, C)
    xs = [x.double().requires_grad_(True) for x in (w_raw, u, k, v)]
    yo = O.wkv4(*xs)
    yo.backward(gy.double())
    y, gw, gu, gk, gv = run_wkv4(R, w_raw, u, k, v, gy)
    for got, want, name in ((y, yo.detach(), "y"), (gw, xs[0].grad, "gw"), (gu, xs[1].grad, "gu"),
                            (gk, xs[2].grad, "gk"), (gv, xs[3].grad, "gv")):
        Hh.assert_close(got, want, Hh.TOL_FP32_STRICT, f"wkv4 {name}")


def test_wkv4_extreme_values_stay_finite(R):
    """k in +-1000 overflows the plain formula; the kernel must not (wkv/run.py:157-161)."""
    g = Hh.gen(1)
    B, T, C = 2, 64, 32
    w_raw, u = Hh.rand(g, C, lo=-5, hi=2), Hh.rand(g, C, lo=-10, hi=10)
    k, v, gy = Hh.rand(g, B, T, C, lo=-1000, hi=1000), Hh.rand(g, B, T, C, lo=-10, hi=10), Hh.randn(g, B, T, C)
    xs = [x.double().requires_grad_(True) for x in (w_raw, u, k, v)]
    yo = O.wkv4(*xs)
    y, gw, gu, gk, gv = run_wkv4(R, w_raw, u, k, v, gy)
    Hh.assert_close(y, yo.detach(), 1e-4, "wkv4 extreme y")
    for t in (gw, gu, gk, gv):
        assert torch.isfinite(t).all()


# ------------------------------------------------------------------ depthwise_conv1d
def run_timex(R, w, k, gy, eps):
    B, C, T = k.shape
    wd, kd, gd = (x.float().to(DEV).contiguous() for x in (w, k, gy))
    x = sentinel(B, C, T)
    R.ops.timex_forward(wd, kd, x, eps, B, C, T)
    gw, gk = sentinel(B, C, T), sentinel(B, C, T)
    R.ops.timex_backward(wd, kd, gd, gw, gk, B, C, T)
    gws, gk2 = sentinel(C, T), sentinel(B, C, T)
    R.ops.timex_backward_reduced(wd, kd, gd, gws, gk2, B, C, T)
    return x, gw.sum(0), gk, gws, gk2


def test_timex_golden(R, golden_dir):
    g = golden(golden_dir, "timex")
    yy = g["y"].clone().requires_grad_(True)
    O.strange_loss(yy).backward()
    x, gw, gk, gws, gk2 = run_timex(R, g["w"], g["k"], yy.grad, float(g["eps"]))
    for got, name in ((x, "y"), (gw, "gw"), (gk, "gk"), (gws, "gw"), (gk2, "gk")):
        Hh.assert_close(got, g[name], Hh.TOL_FP32_STRICT, "timex " + name)


@pytest.mark.parametrize("B,C,T", [(32, 24, 768), (8, 7, 768), (3, 5, 130), (5, 3, 1), (9, 2, 2048), (1, 4, 63)])
def test_timex_oracle(R, B, C, T):
    g = Hh.gen(42)
    w = Hh.randn(g, C, T) / T ** 0.5
    k, gy = Hh.randn(g, B, C, T), Hh.randn(g, B, C, T)
    wl, kl = w.double().requires_grad_(True), k.double().requires_grad_(True)
    yo = O.timex_conv(wl, kl, 0.1)
    yo.backward(gy.double())
    x, gw, gk, gws, gk2 = run_timex(R, w, k, gy, 0.1)
    for got, want, name in ((x, yo.detach(), "x"), (gw, wl.grad, "gw"), (gk, kl.grad, "gk"),
                            (gws, wl.grad, "gw(reduced)"), (gk2, kl.grad, "gk(reduced)")):
        Hh.assert_close(got, want, Hh.TOL_FP32_STRICT, f"timex {name}")


# ------------------------------------------------------------------ RWKV-5 / 5a
def run_wkv5(R, dtype, H, r, k, v, w_raw, u, gy):
    B, T, C = r.shape
    rd, kd, vd, ud, gd = (x.to(dtype).to(DEV).contiguous() for x in (r, k, v, u, gy))
    ew = -torch.exp(w_raw.to(dtype).float()).to(DEV).contiguous()
    eew = torch.exp(ew).contiguous()
    y = sentinel(B, T, C, dtype=dtype)
    R.ops.wkv5_forward(B, T, C, H, rd, kd, vd, eew, ud, y)
    gr, gk, gv = (sentinel(B, T, C, dtype=dtype) for _ in range(3))
    gw, gu = sentinel(B, C, dtype=dtype), sentinel(B, C, dtype=dtype)
    R.ops.wkv5_backward(B, T, C, H, rd, kd, vd, eew, ew, ud, gd, gr, gk, gv, gw, gu)
    return y, gr, gk, gv, gw.float().sum(0), gu.float().sum(0)


def test_wkv5_golden(R, golden_dir):
    g = golden(golden_dir, "wkv5")
    out = run_wkv5(R, torch.float32, int(g["H"]), g["r"], g["k"], g["v"], g["w"], g["u"], g["gy"])
    for got, name in zip(out, ("y", "gr", "gk", "gv", "gw", "gu")):
        Hh.assert_close(got, g[name], Hh.TOL_FP32, "wkv5 " + name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,T,H,N", [(2, 96, 2, 64), (2, 256, 3, 64), (1, 16, 1, 64), (1, 40, 2, 128), (2, 33, 3, 17), (3, 5, 2, 4), (2, 70, 1, 32)])
def test_wkv5_oracle(R, dtype, B, T, H, N):
    g = Hh.gen(42)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.rand(g, H, N, lo=-6, hi=-1), Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w_raw, u)]
    yo = O.wkv5(*xs, H)
    yo.backward(gy.to(dtype).double())
    out = run_wkv5(R, dtype, H, r, k, v, w_raw, u, gy)
    wants = [yo.detach()] + [x.grad for x in xs]
    for got, want, name in zip(out, wants, ("y", "gr", "gk", "gv", "gw", "gu")):
        Hh.assert_close(got, want, Hh.tol_for(dtype), f"wkv5 {name}")


def test_wkv5_strong_decay_falls_back(R):
    """bf16, N = 64, T a multiple of 16 takes the chunked tensor-core kernels; with log-decays below
    -5 per token (w_raw above 1.6) a chunk's cumulative decay is too small to divide by, and the
    general-shape kernels must redo the call."""
    B, T, H, N = 2, 64, 2, 64
    dtype = torch.bfloat16
    g = Hh.gen(3)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.rand(g, H, N, lo=-1, hi=2.5), Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w_raw, u)]
    yo = O.wkv5(*xs, H)
    yo.backward(gy.to(dtype).double())
    out = run_wkv5(R, dtype, H, r, k, v, w_raw, u, gy)
    wants = [yo.detach()] + [x.grad for x in xs]
    for got, want, name in zip(out, wants, ("y", "gr", "gk", "gv", "gw", "gu")):
        assert torch.isfinite(got.float()).all(), name
        Hh.assert_close(got, want, Hh.tol_for(dtype), f"wkv5 strong decay {name}")


@pytest.mark.parametrize("dtype,B,T,H,N,hi", [(torch.bfloat16, 4, 256, 2, 64, -1.0),    # chunked kernels
                                                 (torch.bfloat16, 4, 64, 2, 64, 2.5),       # strong decay: general-shape kernel redoes it
                                                 (torch.bfloat16, 3, 40, 2, 32, -1.0),      # general-shape kernel only
                                                 (torch.float32, 2, 48, 2, 64, -1.0)])
def test_wkv5_parameter_gradients_without_the_bf16_round_trip(R, dtype, B, T, H, N, hi):
    """The fp32 (B,C) partials of gw, gu summed in fp32: at least as close to the oracle as the sum of the
    partials in the activation type, on every kernel path."""
    g = Hh.gen(9)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.rand(g, H, N, lo=-6 if hi < 0 else -1, hi=hi), Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w_raw, u)]
    yo = O.wkv5(*xs, H)
    yo.backward(gy.to(dtype).double())
    rd, kd, vd, ud, gd = (x.to(dtype).to(DEV).contiguous() for x in (r, k, v, u, gy))
    ew = -torch.exp(w_raw.to(dtype).float()).to(DEV).contiguous()
    eew = torch.exp(ew).contiguous()
    gr, gk, gv = (sentinel(B, T, C, dtype=dtype) for _ in range(3))
    gw, gu = sentinel(B, C, dtype=dtype), sentinel(B, C, dtype=dtype)
    gw32, gu32 = sentinel(B, C), sentinel(B, C)
    R.ops.wkv5_backward(B, T, C, H, rd, kd, vd, eew, ew, ud, gd, gr, gk, gv, gw, gu, gw32, gu32)
    sums = torch.empty(2, C, device=DEV)
    R.ops.reduce_batch_partials(gw32, sums[0])
    R.ops.reduce_batch_partials(gu32, sums[1])
    torch.cuda.synchronize()
    for name, got32, part, want in (("gw", sums[0], gw, xs[3].grad), ("gu", sums[1], gu, xs[4].grad)):
        Hh.assert_close(got32, want, Hh.tol_for(dtype), f"wkv5 {name} from fp32 partials")
        e32 = O.err_ratio(want.reshape(-1), got32.double().cpu())
        e16 = O.err_ratio(want.reshape(-1), part.float().sum(0).double().cpu())
        assert e32 <= e16 * 1.05 + 1e-7, (name, e32, e16)


def run_wkv5a(R, dtype, H, r, k, v, w1, u1, w2, u2, gy):
    B, T, C = r.shape
    rd, kd, vd, u1d, u2d, gd = (x.to(dtype).to(DEV).contiguous() for x in (r, k, v, u1, u2, gy))
    ew1 = -torch.exp(w1.to(dtype).float()).to(DEV).contiguous()
    ew2 = -torch.exp(w2.to(dtype).float()).to(DEV).contiguous()
    eew1, eew2 = torch.exp(ew1).contiguous(), torch.exp(ew2).contiguous()
    y = sentinel(B, T, C, dtype=dtype)
    R.ops.wkv5a_forward(B, T, C, H, rd, kd, vd, eew1, u1d, eew2, u2d, y)
    gr, gk, gv = (sentinel(B, T, C, dtype=dtype) for _ in range(3))
    gp = [sentinel(B, C, dtype=dtype) for _ in range(4)]
    R.ops.wkv5a_backward(B, T, C, H, rd, kd, vd, eew1, ew1, u1d, eew2, ew2, u2d, gd, gr, gk, gv, *gp)
    return [y, gr, gk, gv] + [x.float().sum(0) for x in gp]


def test_wkv5a_golden(R, golden_dir):
    g = golden(golden_dir, "wkv5a")
    out = run_wkv5a(R, torch.float32, int(g["H"]), *(g[n] for n in ("r", "k", "v", "w1", "u1", "w2", "u2", "gy")))
    for got, name in zip(out, ("y", "gr", "gk", "gv", "gw1", "gu1", "gw2", "gu2")):
        Hh.assert_close(got, g[name], Hh.TOL_FP32, "wkv5a " + name)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,H,N", [(3, 65, 3, 17), (2, 80, 2, 64), (1, 4, 1, 4)])
def test_wkv5a_oracle(R, dtype, B, T, H, N):
    g = Hh.gen(7)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w1, w2 = Hh.rand(g, H, N, lo=-6, hi=-1), Hh.rand(g, H, N, lo=-6, hi=-1)
    u1, u2, gy = Hh.rand(g, H, N, lo=-1, hi=1), Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w1, u1, w2, u2)]
    yo = O.wkv5a(*xs, H)
    yo.backward(gy.to(dtype).double())
    out = run_wkv5a(R, dtype, H, r, k, v, w1, u1, w2, u2, gy)
    wants = [yo.detach()] + [x.grad for x in xs]
    for got, want, name in zip(out, wants, ("y", "gr", "gk", "gv", "gw1", "gu1", "gw2", "gu2")):
        Hh.assert_close(got, want, Hh.tol_for(dtype), f"wkv5a {name}")


# ------------------------------------------------------------------ RWKV-6
def run_wkv6(R, dtype, H, r, k, v, w_raw, u, gy):
    B, T, C = r.shape
    rd, kd, vd, ud, gd = (x.to(dtype).to(DEV).contiguous() for x in (r, k, v, u, gy))
    ew = -torch.exp(w_raw.to(dtype).float()).to(DEV).contiguous()
    y = sentinel(B, T, C, dtype=dtype)
    R.ops.wkv6_forward(B, T, C, H, rd, kd, vd, ew, ud, y)
    gr, gk, gv, gw = (sentinel(B, T, C, dtype=dtype) for _ in range(4))
    gu = sentinel(B, C, dtype=dtype)
    R.ops.wkv6_backward(B, T, C, H, rd, kd, vd, ew, ud, gd, gr, gk, gv, gw, gu)
    return y, gr, gk, gv, gw, gu.float().sum(0)


def test_wkv6_golden(R, golden_dir):
    g = golden(golden_dir, "wkv6")
    out = run_wkv6(R, torch.float32, int(g["H"]), *(g[n] for n in ("r", "k", "v", "w", "u", "gy")))
    for got, name in zip(out, ("y", "gr", "gk", "gv", "gw", "gu")):
        Hh.assert_close(got, g[name], Hh.TOL_FP32, "wkv6 " + name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,T,H,N", [(2, 300, 2, 64), (2, 256, 2, 64), (1, 16, 1, 64), (2, 32, 3, 64), (2, 7, 2, 4), (1, 50, 1, 128), (2, 41, 3, 17)])
def test_wkv6_oracle(R, dtype, B, T, H, N):
    """T = 300 is beyond what the reference backward can run (wkv6/run.py:51)."""
    g = Hh.gen(42)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.randn(g, B, T, C) - 3.0, Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w_raw, u)]
    yo = O.wkv6(*xs, H)
    yo.backward(gy.to(dtype).double())
    out = run_wkv6(R, dtype, H, r, k, v, w_raw, u, gy)
    wants = [yo.detach()] + [x.grad for x in xs]
    for got, want, name in zip(out, wants, ("y", "gr", "gk", "gv", "gw", "gu")):
        Hh.assert_close(got, want, Hh.tol_for(dtype), f"wkv6 {name}")


# ------------------------------------------------------------------ RWKV-6 with state
def run_wkv6state(R, dtype, H, r, k, v, w_raw, u, s, gy):
    B, T, C = r.shape
    N = C // H
    rd, kd, vd, wd, ud, sd, gd = (x.to(dtype).to(DEV).contiguous() for x in (r, k, v, w_raw, u, s, gy))
    y = sentinel(B, T, C, dtype=dtype)
    R.ops.wkv6state_forward(B, T, C, H, rd, kd, vd, wd, ud, sd, y)
    gr, gk, gv, gw = (sentinel(B, T, C, dtype=dtype) for _ in range(4))
    gu, gs = sentinel(B, C, dtype=dtype), sentinel(B, H, N, N, dtype=dtype)
    R.ops.wkv6state_backward(B, T, C, H, rd, kd, vd, wd, ud, sd, gd, gr, gk, gv, gw, gu, gs)
    return y, gr, gk, gv, gw, gu.float().sum(0), gs


def test_wkv6state_golden(R, golden_dir):
    g = golden(golden_dir, "wkv6state")
    out = run_wkv6state(R, torch.float32, int(g["H"]), *(g[n] for n in ("r", "k", "v", "w", "u", "s", "gy")))
    for got, name in zip(out, ("y", "gr", "gk", "gv", "gw", "gu", "gs")):
        Hh.assert_close(got, g[name], Hh.TOL_FP32, "wkv6state " + name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,T,H,N", [(2, 200, 2, 64), (2, 192, 2, 64), (1, 16, 2, 64), (3, 7, 2, 4)])
def test_wkv6state_oracle(R, dtype, B, T, H, N):
    g = Hh.gen(42)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.randn(g, B, T, C) - 3.0, Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    s = 0.1 * Hh.randn(g, B, H, N, N)
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w_raw, u, s)]
    yo = O.wkv6(*xs[:5], H, s0=xs[5])
    yo.backward(gy.to(dtype).double())
    out = run_wkv6state(R, dtype, H, r, k, v, w_raw, u, s, gy)
    wants = [yo.detach()] + [x.grad for x in xs]
    for got, want, name in zip(out, wants, ("y", "gr", "gk", "gv", "gw", "gu", "gs")):
        Hh.assert_close(got, want, Hh.tol_for(dtype), f"wkv6state {name}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_wkv6state_ex_oracle(R, dtype):
    """fp32 state in, final state out, gradient of the final state in (state passing)."""
    B, T, H, N = 2, 160, 2, 64
    g = Hh.gen(5)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.randn(g, B, T, C) - 5.0, Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    s0, dsT = 0.1 * Hh.randn(g, B, H, N, N), Hh.randn(g, B, H, N, N)
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w_raw, u)] + [s0.double().requires_grad_(True)]
    yo, sTo = O.wkv6(*xs[:5], H, s0=xs[5], return_state=True)
    torch.autograd.backward([yo, sTo], [gy.to(dtype).double(), dsT.double()])
    rd, kd, vd, wd, ud, gd = (x.to(dtype).to(DEV).contiguous() for x in (r, k, v, w_raw, u, gy))
    s0d, dsTd = s0.to(DEV), dsT.to(DEV)
    y, sT = sentinel(B, T, C, dtype=dtype), sentinel(B, H, N, N)
    R.ops.wkv6state_forward_ex(B, T, C, H, rd, kd, vd, wd, ud, s0d, y, sT)
    gr, gk, gv, gw = (sentinel(B, T, C, dtype=dtype) for _ in range(4))
    gu, ds0 = sentinel(B, C, dtype=dtype), sentinel(B, H, N, N)
    R.ops.wkv6state_backward_ex(B, T, C, H, rd, kd, vd, wd, ud, s0d, gd, dsTd, gr, gk, gv, gw, gu, ds0)
    tol = Hh.tol_for(dtype)
    wants = [yo.detach(), sTo.detach()] + [x.grad for x in xs]
    for got, want, name in zip((y, sT, gr, gk, gv, gw, gu.float().sum(0), ds0), wants,
                               ("y", "sT", "gr", "gk", "gv", "gw", "gu", "ds0")):
        Hh.assert_close(got, want, tol, f"wkv6state_ex {name}")


@pytest.mark.parametrize("shift", [2.0, 5.0])
def test_wkv6_strong_decay_falls_back(R, shift):
    """bf16, N = 64, T a multiple of 16 takes the chunked tensor-core kernels, which divide by the
    cumulative decay of a chunk.  With decays this strong (log-decay down to -e^6 per token) that
    form is unusable: the kernel must notice and the general-shape kernels must redo the call."""
    B, T, H, N = 2, 128, 2, 64
    dtype = torch.bfloat16
    g = Hh.gen(9)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.randn(g, B, T, C) + shift, Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w_raw, u)]
    yo = O.wkv6(*xs, H)
    yo.backward(gy.to(dtype).double())
    out = run_wkv6(R, dtype, H, r, k, v, w_raw, u, gy)
    wants = [yo.detach()] + [x.grad for x in xs]
    for got, want, name in zip(out, wants, ("y", "gr", "gk", "gv", "gw", "gu")):
        assert torch.isfinite(got.float()).all(), name
        if name == "gw" and shift > 3:
            continue   # e^5 and more per token: the decay gradient is below what bf16 inputs resolve
        Hh.assert_close(got, want, Hh.tol_for(dtype), f"wkv6 strong decay {name}")


def test_wkv6_strong_decay_in_one_unit_only(R):
    """One (batch, head) unit of six has a decay too strong for the chunked form: only that unit is redone by
    the general-shape kernels (one flag per unit), every unit's results must be right."""
    B, T, H, N = 3, 128, 2, 64
    dtype = torch.bfloat16
    g = Hh.gen(19)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.randn(g, B, T, C) - 3.0, Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    w_raw[1, 32:64, N:2 * N] += 5.5          # unit (b=1, h=1), tokens 32-63
    xs = [x.to(dtype).double().requires_grad_(True) for x in (r, k, v, w_raw, u)]
    yo = O.wkv6(*xs, H)
    yo.backward(gy.to(dtype).double())
    out = run_wkv6(R, dtype, H, r, k, v, w_raw, u, gy)
    wants = [yo.detach()] + [x.grad for x in xs]
    for got, want, name in zip(out, wants, ("y", "gr", "gk", "gv", "gw", "gu")):
        assert torch.isfinite(got.float()).all(), name
        Hh.assert_close(got, want, Hh.tol_for(dtype), f"wkv6, one unit with a strong decay: {name}")


# ------------------------------------------------------------------ RWKV-7
def run_wkv7(R, dtype, H, inp, use_s0, use_sT, chunk=16):
    B, T, C = inp["r"].shape
    N = C // H
    d = {n: inp[n].to(dtype).to(DEV).view(B, T, H, N).contiguous() for n in ("r", "w", "k", "v", "a", "b", "dy")}
    s0 = inp["s0"].float().to(DEV).contiguous() if use_s0 else None
    dsT = inp["dsT"].float().to(DEV).contiguous() if use_sT else None
    y = sentinel(B, T, H, N, dtype=dtype)
    sT = sentinel(B, H, N, N) if use_sT else None
    s = sentinel(B, H, T // chunk, N, N)
    sa = sentinel(B, T, H, N)
    R.ops.wkv7_forward(s0, d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], y, sT, s, sa)
    grads = [sentinel(B, T, H, N, dtype=dtype) for _ in range(6)]
    ds0 = sentinel(B, H, N, N) if use_s0 else None
    R.ops.wkv7_backward(d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], d["dy"], dsT, s, sa, ds0, *grads)
    out = dict(y=y, sT=sT, ds0=ds0)
    out.update({n: x for n, x in zip(("dr", "dw", "dk", "dv", "da", "db"), grads)})
    return out


@pytest.mark.parametrize("variant,use_s0,use_sT", [("wkv7_clampw", False, False), ("wkv7_state_clampw", True, False),
                                                   ("wkv7_statepassing_clampw", True, True)])
def test_wkv7_golden_fp32(R, golden_dir, variant, use_s0, use_sT):
    g = golden(golden_dir, variant)
    H = int(g["H"])
    out = run_wkv7(R, torch.float32, H, g, use_s0, use_sT)
    names = ["y", "dr", "dw", "dk", "dv", "da", "db"] + (["ds0"] if use_s0 else []) + (["sT"] if use_sT else [])
    for n in names:
        Hh.assert_close(out[n], g[n], Hh.TOL_FP32, f"{variant} {n}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,T,H,N", [(2, 64, 2, 16), (2, 128, 2, 64), (1, 32, 1, 128), (1, 48, 2, 32)])
@pytest.mark.parametrize("use_s0,use_sT", [(True, True), (False, False), (True, False)])
def test_wkv7_oracle(R, dtype, B, T, H, N, use_s0, use_sT):
    inp = Hh.v7_inputs(B, T, H, N)
    inp64 = {n: (x.to(dtype).double() if n not in ("s0", "dsT") else x.double()) for n, x in inp.items()}
    want = Hh.v7_oracle(inp64, H, use_s0=use_s0, use_dsT=use_sT)
    out = run_wkv7(R, dtype, H, inp, use_s0, use_sT)
    tol = Hh.tol_for(dtype)
    names = ["y", "dr", "dw", "dk", "dv", "da", "db"] + (["ds0"] if use_s0 else []) + (["sT"] if use_sT else [])
    for n in names:
        Hh.assert_close(out[n], want[n], tol, f"wkv7 {n}")


def test_wkv7_chunk_len_other_than_16(R):
    """The checkpoint stride is a runtime value (the reference bakes -D_CHUNK_LEN_ in)."""
    B, T, H, N = 1, 96, 2, 64
    inp = Hh.v7_inputs(B, T, H, N, seed=3)
    inp64 = {n: (x.to(torch.bfloat16).double() if n not in ("s0", "dsT") else x.double()) for n, x in inp.items()}
    want = Hh.v7_oracle(inp64, H)
    for chunk in (8, 32):
        out = run_wkv7(R, torch.bfloat16, H, inp, True, True, chunk=chunk)
        for n in ("y", "dr", "dw", "dk", "dv", "da", "db", "ds0", "sT"):
            Hh.assert_close(out[n], want[n], Hh.TOL_BF16, f"wkv7 chunk {chunk} {n}")


def test_wkv7_state_passing_composes(R):
    """Two segments with the state handed over reproduce one pass over the whole sequence."""
    B, T, H, N = 2, 128, 2, 64
    inp = Hh.v7_inputs(B, T, H, N, seed=11)
    d = {n: inp[n].to(torch.bfloat16).to(DEV).view(B, T, H, N).contiguous() for n in ("r", "w", "k", "v", "a", "b")}
    s0 = inp["s0"].to(DEV)

    def fwd(lo, hi, s_in):
        seg = {n: x[:, lo:hi].contiguous() for n, x in d.items()}
        y = sentinel(B, hi - lo, H, N, dtype=torch.bfloat16)
        sT = sentinel(B, H, N, N)
        R.ops.wkv7_forward(s_in, seg["r"], seg["w"], seg["k"], seg["v"], seg["a"], seg["b"], y, sT, None, None)
        return y, sT

    y, sT = fwd(0, T, s0)
    # a cut on a 32-token boundary keeps the kernels' chunks where they are: bit-identical
    ya, sm = fwd(0, 64, s0)
    yb, sT2 = fwd(64, T, sm)
    assert torch.equal(torch.cat([ya, yb], 1), y)
    assert torch.equal(sT2, sT)
    # any other multiple of 16 regroups the tokens into different chunks: equal to rounding
    ya, sm = fwd(0, 48, s0)
    yb, sT3 = fwd(48, T, sm)
    assert O.err_ratio(y.double().cpu(), torch.cat([ya, yb], 1).double().cpu()) < 4e-3   # two bf16 roundings
    assert O.err_ratio(sT.double().cpu(), sT3.double().cpu()) < 1e-3


def test_wkv6_chunked_calls_on_two_streams(R):
    """Two chunked RWKV-6 calls in flight on different streams, one of them with decays that force
    the fall-back: each stream has its own device flag, so neither disturbs the other -- however many
    calls are queued (100 per stream here, more than any fixed ring of flags would hold)."""
    B, T, H, N = 2, 128, 2, 64
    dtype = torch.bfloat16
    C = H * N
    results = {}
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    cases = {}
    for idx, shift in enumerate((-3.0, 5.0)):
        g = Hh.gen(20 + idx)
        r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
        w_raw, u = Hh.randn(g, B, T, C) + shift, Hh.rand(g, H, N, lo=-1, hi=1)
        xs = [x.to(dtype).double() for x in (r, k, v, w_raw, u)]
        cases[idx] = (O.wkv6(*xs, H), [x.to(dtype).to(DEV).contiguous() for x in (r, k, v)],
                      (-torch.exp(w_raw.to(dtype).float())).to(DEV).contiguous(), u.to(dtype).to(DEV).contiguous())
    torch.cuda.synchronize()
    for rep in range(100):
        for idx, st in enumerate(streams):
            _, (rd, kd, vd), ew, ud = cases[idx]
            with torch.cuda.stream(st):
                y = sentinel(B, T, C, dtype=dtype)
                R.ops.wkv6_forward(B, T, C, H, rd, kd, vd, ew, ud, y)
                results[idx] = y
    torch.cuda.synchronize()
    for idx in cases:
        Hh.assert_close(results[idx], cases[idx][0], Hh.tol_for(dtype), f"wkv6 stream {idx}")


@pytest.mark.parametrize("dtype,N", [(torch.bfloat16, 64), (torch.float32, 64), (torch.bfloat16, 32)])
def test_wkv7_state_update_decoding_and_prompt(R, dtype, N):
    """Inference entry point: a prompt (any length) followed by single-token steps, state updated in place,
    equals the fp64 formula on the concatenated sequence."""
    B, H = 2, 3
    lens = [96, 5, 1, 1, 1]
    T = sum(lens)
    inp = Hh.v7_inputs(B, T, H, N, seed=9)
    x64 = {n: inp[n].to(dtype).double() for n in ("r", "w", "k", "v", "a", "b")}
    y64, sT64 = O.wkv7(*(x64[n] for n in ("r", "w", "k", "v", "a", "b")), H, s0=inp["s0"].double())
    d = {n: inp[n].to(dtype).to(DEV).view(B, T, H, N).contiguous() for n in ("r", "w", "k", "v", "a", "b")}
    state = inp["s0"].to(DEV).clone()
    ys, lo = [], 0
    for L in lens:
        seg = {n: x[:, lo:lo + L].contiguous() for n, x in d.items()}
        y = sentinel(B, L, H, N, dtype=dtype)
        R.ops.wkv7_state_update(state, seg["r"], seg["w"], seg["k"], seg["v"], seg["a"], seg["b"], y)
        ys.append(y)
        lo += L
    torch.cuda.synchronize()
    tol = Hh.tol_for(dtype)
    Hh.assert_close(torch.cat(ys, 1).view(B, T, H * N), y64, tol, "y")
    Hh.assert_close(state, sT64, tol, "state")
