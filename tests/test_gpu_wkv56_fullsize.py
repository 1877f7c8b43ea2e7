"""RWKV-5 and RWKV-6-with-state chunked kernels at the sizes that are benchmarked (RWKV-5 bf16 B8 T4096 C4096,
RWKV-6 state bf16 B16 T4096 C4096: 512 / 1024 thread blocks, several waves per SM).

The fp64 oracle runs on a few (batch, head) units only: units are independent, so a unit of the full launch
must equal the oracle on that unit's inputs (one batch row, one head); the per-row partials of the parameter
gradients gw / gu of that unit are the oracle's parameter gradients for that unit alone."""
import pytest
import torch

from oracle import wkv_oracle as O
from tests import helpers as Hh

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16
PICKS = {8: [(0, 0), (3, 37), (7, 63)], 16: [(0, 0), (6, 21), (15, 63)]}   # first, one of a middle wave, last


def _draw(B, T, H, N, seed, per_token_decay):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    C = H * N
    mk = lambda sc=1.0: torch.randn(B, T, C, generator=g, device=DEV) * sc
    d = {"r": mk(0.5).to(BF), "k": mk(0.5).to(BF), "v": mk(0.5).to(BF), "gy": mk().to(BF)}
    if per_token_decay:
        d["w_raw"] = (mk() - 3.0).to(BF)                                                    # (B,T,C)
    else:
        d["w_raw"] = (torch.rand(H, N, generator=g, device=DEV) * 5.0 - 6.0).to(BF)         # (H,N) in [-6,-1]
    d["u"] = (torch.rand(H, N, generator=g, device=DEV) * 2.0 - 1.0).to(BF)
    return d


def _unit(d, b, h, N, names):
    sl = slice(h * N, (h + 1) * N)
    return [d[n][b : b + 1, :, sl].double().cpu().contiguous().requires_grad_(True) for n in names]


def test_rwkv5_benchmark_size_units_against_oracle():
    import rwkv_cuda_b200 as R
    B, T, H, N = 8, 4096, 64, 64
    C = H * N
    d = _draw(B, T, H, N, seed=42, per_token_decay=False)
    ew = -torch.exp(d["w_raw"].float()).contiguous()
    eew = torch.exp(ew).contiguous()
    y = torch.empty(B, T, C, dtype=BF, device=DEV)
    R.ops.wkv5_forward(B, T, C, H, d["r"], d["k"], d["v"], eew, d["u"], y)
    gr, gk, gv = (torch.empty_like(y) for _ in range(3))
    gw, gu = torch.empty(B, C, dtype=BF, device=DEV), torch.empty(B, C, dtype=BF, device=DEV)
    R.ops.wkv5_backward(B, T, C, H, d["r"], d["k"], d["v"], eew, ew, d["u"], d["gy"], gr, gk, gv, gw, gu)
    torch.cuda.synchronize()
    for t in (y, gr, gk, gv, gw, gu):
        assert torch.isfinite(t.float()).all()
    rep = []
    for b, h in PICKS[B]:
        sl = slice(h * N, (h + 1) * N)
        r1, k1, v1 = _unit(d, b, h, N, ("r", "k", "v"))
        w1 = d["w_raw"][h : h + 1].double().cpu().requires_grad_(True)
        u1 = d["u"][h : h + 1].double().cpu().requires_grad_(True)
        yo = O.wkv5(r1, k1, v1, w1, u1, 1)
        yo.backward(d["gy"][b : b + 1, :, sl].double().cpu())
        pairs = [(y[b, :, sl], yo.detach()[0], "y"), (gr[b, :, sl], r1.grad[0], "gr"), (gk[b, :, sl], k1.grad[0], "gk"),
                 (gv[b, :, sl], v1.grad[0], "gv"), (gw[b, sl], w1.grad[0], "gw"), (gu[b, sl], u1.grad[0], "gu")]
        for got, want, name in pairs:
            _, e = Hh.assert_close(got, want, Hh.TOL_BF16, f"wkv5 {name} of unit ({b},{h})")
            rep.append(f"({b},{h}) {name}: rms {e:.2e}")
    print("\n".join(rep))


def test_rwkv6_state_benchmark_size_units_against_oracle():
    import rwkv_cuda_b200 as R
    B, T, H, N = 16, 4096, 64, 64
    C = H * N
    d = _draw(B, T, H, N, seed=43, per_token_decay=True)
    g = torch.Generator(device=DEV)
    g.manual_seed(7)
    s0 = 0.1 * torch.randn(B, H, N, N, generator=g, device=DEV)
    dsT = torch.randn(B, H, N, N, generator=g, device=DEV)
    y, sT = torch.empty(B, T, C, dtype=BF, device=DEV), torch.empty_like(s0)
    R.ops.wkv6state_forward_ex(B, T, C, H, d["r"], d["k"], d["v"], d["w_raw"], d["u"], s0, y, sT)
    gr, gk, gv, gw = (torch.empty_like(y) for _ in range(4))
    gu, ds0 = torch.empty(B, C, dtype=BF, device=DEV), torch.empty_like(s0)
    R.ops.wkv6state_backward_ex(B, T, C, H, d["r"], d["k"], d["v"], d["w_raw"], d["u"], s0, d["gy"], dsT, gr, gk, gv, gw,
                                gu, ds0)
    torch.cuda.synchronize()
    for t in (y, sT, gr, gk, gv, gw, gu, ds0):
        assert torch.isfinite(t.float()).all()
    rep = []
    for b, h in PICKS[B]:
        sl = slice(h * N, (h + 1) * N)
        r1, k1, v1, w1 = _unit(d, b, h, N, ("r", "k", "v", "w_raw"))
        u1 = d["u"][h : h + 1].double().cpu().requires_grad_(True)
        s1 = s0[b : b + 1, h : h + 1].double().cpu().requires_grad_(True)
        yo, sTo = O.wkv6(r1, k1, v1, w1, u1, 1, s0=s1, return_state=True)
        torch.autograd.backward([yo, sTo], [d["gy"][b : b + 1, :, sl].double().cpu(), dsT[b : b + 1, h : h + 1].double().cpu()])
        pairs = [(y[b, :, sl], yo.detach()[0], "y"), (sT[b, h], sTo.detach()[0, 0], "sT"), (gr[b, :, sl], r1.grad[0], "gr"),
                 (gk[b, :, sl], k1.grad[0], "gk"), (gv[b, :, sl], v1.grad[0], "gv"), (gw[b, :, sl], w1.grad[0], "gw"),
                 (gu[b, sl], u1.grad[0], "gu"), (ds0[b, h], s1.grad[0, 0], "ds0")]
        for got, want, name in pairs:
            _, e = Hh.assert_close(got, want, Hh.TOL_BF16, f"wkv6state {name} of unit ({b},{h})")
            rep.append(f"({b},{h}) {name}: rms {e:.2e}")
    print("\n".join(rep))
