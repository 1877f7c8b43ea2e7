"""The oracle against the golden vectors made from the reference's own formula functions
(tests/golden/make_golden.py), and the oracle's independent restatements against each other."""
import os

import numpy as np
import pytest
import torch

from oracle import wkv_oracle as O

TOL = 1e-9  # fp64 round-off over these tiny shapes


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: torch.from_numpy(np.asarray(z[k])) for k in z.files}


def leafs(g, *names):
    return [g[n].clone().requires_grad_(True) for n in names]


def check(got, want, what):
    err = O.max_err(want, got.reshape(want.shape))
    assert err < TOL, f"{what}: max err {err:.3e}"


def test_wkv4(golden_dir):
    g = load(golden_dir, "wkv4")
    w, u, k, v = leafs(g, "w", "u", "k", "v")
    y = O.wkv4(w, u, k, v)
    check(y, g["y"], "y")
    check(O.wkv4_bruteforce(w, u, k, v), g["y"], "y brute")
    O.strange_loss(y).backward()
    for got, name in ((w.grad, "gw"), (u.grad, "gu"), (k.grad, "gk"), (v.grad, "gv")):
        check(got, g[name], name)


def test_timex(golden_dir):
    g = load(golden_dir, "timex")
    w, k = leafs(g, "w", "k")
    y = O.timex(w, k, float(g["eps"]))
    check(y, g["y"], "y")
    check(O.timex_conv(w, k, float(g["eps"])), g["y"], "y conv")
    O.strange_loss(y).backward()
    check(w.grad, g["gw"], "gw")
    check(k.grad, g["gk"], "gk")


def test_wkv5(golden_dir):
    g = load(golden_dir, "wkv5")
    H = int(g["H"])
    r, k, v, w, u = leafs(g, "r", "k", "v", "w", "u")
    y = O.wkv5(r, k, v, w, u, H)
    check(y, g["y"], "y")
    check(O.wkv5_bruteforce(r, k, v, w, u, H), g["y"], "y brute")
    y.backward(g["gy"])
    for x, name in ((r, "gr"), (k, "gk"), (v, "gv"), (w, "gw"), (u, "gu")):
        check(x.grad, g[name], name)


def test_wkv5a(golden_dir):
    g = load(golden_dir, "wkv5a")
    H = int(g["H"])
    xs = leafs(g, "r", "k", "v", "w1", "u1", "w2", "u2")
    y = O.wkv5a(*xs, H)
    check(y, g["y"], "y")
    y.backward(g["gy"])
    for x, name in zip(xs, ("gr", "gk", "gv", "gw1", "gu1", "gw2", "gu2")):
        check(x.grad, g[name], name)


def test_wkv5a_reduces_to_wkv5():
    torch.manual_seed(1)
    B, T, H, N = 2, 6, 2, 3
    r, k, v = (torch.randn(B, T, H * N, dtype=torch.float64) for _ in range(3))
    w, u = torch.randn(H, N, dtype=torch.float64), torch.randn(H, N, dtype=torch.float64)
    w2 = torch.full((H, N), -40.0, dtype=torch.float64)   # exp(-exp(-40)) == 1
    y5a = O.wkv5a(r, k, v, w, u, w2, torch.zeros(H, N, dtype=torch.float64), H)
    check(y5a, O.wkv5(r, k, v, w, u, H), "wkv5a->wkv5")


def test_wkv6(golden_dir):
    g = load(golden_dir, "wkv6")
    H = int(g["H"])
    r, k, v, w, u = leafs(g, "r", "k", "v", "w", "u")
    y = O.wkv6(r, k, v, w, u, H)
    check(y, g["y"], "y")
    check(O.wkv6_bruteforce(r, k, v, w, u, H), g["y"], "y brute")
    y.backward(g["gy"])
    for x, name in ((r, "gr"), (k, "gk"), (v, "gv"), (w, "gw"), (u, "gu")):
        check(x.grad, g[name], name)


def test_wkv6state(golden_dir):
    g = load(golden_dir, "wkv6state")
    H = int(g["H"])
    r, k, v, w, u, s = leafs(g, "r", "k", "v", "w", "u", "s")
    y = O.wkv6(r, k, v, w, u, H, s0=s)
    check(y, g["y"], "y")
    check(O.wkv6_bruteforce(r, k, v, w, u, H, s0=s), g["y"], "y brute")
    y.backward(g["gy"])
    for x, name in ((r, "gr"), (k, "gk"), (v, "gv"), (w, "gw"), (u, "gu"), (s, "gs")):
        check(x.grad, g[name], name)


def test_wkv6_state_passing_composes():
    """Running two segments with the state handed over equals one run over the whole sequence."""
    torch.manual_seed(2)
    B, T, H, N = 2, 10, 2, 4
    r, k, v = (torch.randn(B, T, H * N, dtype=torch.float64) for _ in range(3))
    w = torch.randn(B, T, H * N, dtype=torch.float64) - 2
    u = torch.randn(H, N, dtype=torch.float64)
    s0 = torch.randn(B, H, N, N, dtype=torch.float64)
    y, sT = O.wkv6(r, k, v, w, u, H, s0=s0, return_state=True)
    ya, sm = O.wkv6(r[:, :4], k[:, :4], v[:, :4], w[:, :4], u, H, s0=s0, return_state=True)
    yb, sT2 = O.wkv6(r[:, 4:], k[:, 4:], v[:, 4:], w[:, 4:], u, H, s0=sm, return_state=True)
    check(torch.cat([ya, yb], 1), y, "y")
    check(sT2, sT, "sT")


@pytest.mark.parametrize("variant", ["wkv7_clampw", "wkv7_state_clampw", "wkv7_statepassing_clampw"])
def test_wkv7(golden_dir, variant):
    g = load(golden_dir, variant)
    H = int(g["H"])
    r, w, k, v, a, b = leafs(g, "r", "w", "k", "v", "a", "b")
    s0 = g["s0"].clone().requires_grad_(True) if "s0" in g else None
    y, sT = O.wkv7(r, w, k, v, a, b, H, s0=s0)
    check(y, g["y"], "y")
    if "sT" in g:
        check(sT, g["sT"], "sT")
        torch.autograd.backward([y, sT], [g["dy"], g["dsT"]])
    else:
        y.backward(g["dy"])
    for x, name in ((r, "dr"), (w, "dw"), (k, "dk"), (v, "dv"), (a, "da"), (b, "db")):
        check(x.grad, g[name], name)
    if s0 is not None:
        check(s0.grad, g["ds0"], "ds0")


def test_wkv7_decay_is_soft_clamped():
    """decay = exp(-e^{-0.5} sigmoid(w_raw)) stays in (exp(-e^{-0.5}), 1): what makes the
    backward's division by the decay safe (rwkv7_statepassing_clampw.cu:16,45)."""
    w_raw = torch.linspace(-30, 30, 101, dtype=torch.float64)
    d = torch.exp(-torch.exp(-torch.nn.functional.softplus(-w_raw) - 0.5))
    assert torch.allclose(d, torch.exp(O.W_SCALE * torch.sigmoid(w_raw)), atol=1e-14)
    assert d.min() > 0.545 and d.max() <= 1.0
