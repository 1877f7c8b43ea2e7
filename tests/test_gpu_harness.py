"""GPU: the reference harnesses' flows (load(...) + autograd.Function + the 'strange loss'),
run through the stand-ins, against autograd through the fp64 oracle."""
import pytest
import torch
import torch.nn.functional as F

from oracle import wkv_oracle as O
from tests import helpers as Hh

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _leaf(x, dtype=None):
    x = x.to(DEV)
    if dtype is not None:
        x = x.to(dtype)
    return x.detach().requires_grad_(True)


def test_rwkv7_state_passing_harness_flow():
    """rwkv7_cuda_benchmark_state_passing.py: load(..., is_python_module=False), the OP class calling
    torch.ops.rwkv7_statepassing_clampw.*, LOSS with a state term, harness input distributions."""
    import rwkv_cuda_b200 as R
    B, T, C, N = 2, 64, 128, 64
    H = C // N
    flags = ["-res-usage", f"-D_N_={N}", "-D_CHUNK_LEN_=16", "--use_fast_math", "-O3", "-Xptxas -O3"]
    R.load(name="rwkv7_statepassing_clampw", sources=["cuda/rwkv7_statepassing_clampw.cu", "cuda/rwkv7_statepassing_clampw.cpp"],
           is_python_module=False, verbose=True, extra_cuda_cflags=flags)

    class OP(torch.autograd.Function):          # as in the harness (:75-99)
        @staticmethod
        def forward(ctx, s0, r, w, k, v, a, b):
            B, T, H, N = r.shape
            y, sT = torch.empty_like(v), torch.empty_like(s0)
            s = torch.empty(B, H, T // 16, N, N, dtype=torch.float32, device=w.device)
            sa = torch.empty(B, T, H, N, dtype=torch.float32, device=w.device)
            torch.ops.rwkv7_statepassing_clampw.forward(s0, r, w, k, v, a, b, y, sT, s, sa)
            ctx.save_for_backward(r, w, k, v, a, b, s, sa)
            return y.view(B, T, H * N), sT

        @staticmethod
        def backward(ctx, dy, dsT):
            r, w, k, v, a, b, s, sa = ctx.saved_tensors
            ds0, dr, dw, dk, dv, da, db = [torch.empty_like(x) for x in [dsT, r, w, k, v, a, b]]
            torch.ops.rwkv7_statepassing_clampw.backward(r, w, k, v, a, b, dy.contiguous(), dsT.contiguous(), s, sa,
                                                          ds0, dr, dw, dk, dv, da, db)
            return ds0, dr, dw, dk, dv, da, db

    g = Hh.gen(42)
    r, k, v = (Hh.rand(g, B, T, C, lo=-1, hi=1) * 3 for _ in range(3))
    w = Hh.rand(g, B, T, C, lo=-6, hi=0)
    a = F.normalize(Hh.rand(g, B, T, C, lo=-1, hi=1) * 2, dim=-1, p=2.0)
    b = F.normalize(Hh.rand(g, B, T, C, lo=-1, hi=1) * 2, dim=-1, p=2.0)
    s = Hh.rand(g, B, H, N, N, lo=-1, hi=1) * 10
    bf = torch.bfloat16

    def loss(y, sT):
        return ((y * y) - torch.tanh(y)).sum() + 16 * (sT * sT + torch.tanh(sT)).sum()

    ref_in = [x.to(bf).double().requires_grad_(True) for x in (r, w, k, v, a, b)]
    s64 = s.double().requires_grad_(True)
    y64, sT64 = O.wkv7(*ref_in, H, s0=s64)
    loss(y64, sT64).backward()

    xs = [_leaf(x, bf) for x in (r, w, k, v, a, b)]
    sd = _leaf(s)
    y, sT = OP.apply(sd, *(x.view(B, T, H, N) for x in xs))
    loss(y.float(), sT).backward()
    Hh.assert_close(y, y64.detach(), Hh.TOL_BF16, "y")
    Hh.assert_close(sT, sT64.detach(), Hh.TOL_BF16, "sT")
    Hh.assert_close(sd.grad, s64.grad, Hh.TOL_BF16, "g_s")
    for name, x, x64 in zip("rwkvab", xs, ref_in):
        Hh.assert_close(x.grad, x64.grad, Hh.TOL_BF16, "g_" + name)


def test_functions_autograd_classes():
    """WKV, TimeX, WKV_5, WKV_5A, WKV_6, WKV_6STATE through autograd with the harness loss."""
    import rwkv_cuda_b200 as R
    Fn = R.functions
    g = Hh.gen(3)
    # RWKV-4 (wkv/run.py:147-234)
    B, T, C = 3, 40, 24
    w, u, k, v = (Hh.rand(g, *s, lo=-1, hi=1) for s in ((C,), (C,), (B, T, C), (B, T, C)))
    ls = [_leaf(x) for x in (w, u, k, v)]
    l64 = [x.double().requires_grad_(True) for x in (w, u, k, v)]
    O.strange_loss(Fn.WKV.apply(B, T, C, *ls)).backward()
    O.strange_loss(O.wkv4(*l64)).backward()
    for a_, b_, n in zip(ls, l64, "wukv"):
        Hh.assert_close(a_.grad, b_.grad, 2e-5, "wkv4 g" + n)
    # depthwise_conv1d (depthwise_conv1d/run.py:135-184)
    B, C, T = 8, 6, 64
    w, k = torch.rand(C, T, generator=g), torch.rand(B, C, T, generator=g)
    ls, l64 = [_leaf(w), _leaf(k)], [w.double().requires_grad_(True), k.double().requires_grad_(True)]
    O.strange_loss(Fn.TimeX.apply(ls[0], ls[1], B, C, T, 0.1)).backward()
    O.strange_loss(O.timex(l64[0], l64[1], 0.1)).backward()
    for a_, b_, n in zip(ls, l64, "wk"):
        Hh.assert_close(a_.grad, b_.grad, 2e-5, "timex g" + n)
    # multi-head family, bf16
    bf = torch.bfloat16
    B, T, H, N = 2, 48, 2, 64
    C = H * N
    r, k, v = (Hh.rand(g, B, T, C, lo=-1, hi=1) for _ in range(3))
    wh, uh = Hh.rand(g, H, N, lo=-6, hi=-1), Hh.rand(g, H, N, lo=-1, hi=1)
    w2, u2 = Hh.rand(g, H, N, lo=-6, hi=-1), Hh.rand(g, H, N, lo=-1, hi=1)
    wt = Hh.randn(g, B, T, C) - 3
    s = 0.1 * Hh.randn(g, B, H, N, N)

    def check(name, out_fn, ora_fn, tensors):
        ls = [_leaf(x, bf) for x in tensors]
        l64 = [x.to(bf).double().requires_grad_(True) for x in tensors]
        y = out_fn(*ls)
        y64 = ora_fn(*l64)
        O.strange_loss(y.float()).backward()
        # the oracle gets the gradient the bf16 run actually saw, so only the operator is compared
        yy = y.detach().float().cpu().double().requires_grad_(True)
        O.strange_loss(yy).backward()
        y64.backward(yy.grad.to(bf).double().view_as(y64))
        Hh.assert_close(y, y64.detach(), Hh.TOL_BF16, name + " y")
        for i, (a_, b_) in enumerate(zip(ls, l64)):
            Hh.assert_close(a_.grad, b_.grad, 3e-2, f"{name} grad {i}")

    check("WKV_5", lambda r, k, v, w, u: Fn.WKV_5.apply(B, T, C, H, r, k, v, w, u),
          lambda r, k, v, w, u: O.wkv5(r, k, v, w, u, H), (r, k, v, wh, uh))
    check("WKV_5A", lambda *xs: Fn.WKV_5A.apply(*xs), lambda *xs: O.wkv5a(*xs, H), (r, k, v, wh, uh, w2, u2))
    check("WKV_6", lambda r, k, v, w, u: Fn.WKV_6.apply(B, T, C, H, r, k, v, w, u),
          lambda r, k, v, w, u: O.wkv6(r, k, v, w, u, H), (r, k, v, wt, uh))
    check("WKV_6STATE", lambda r, k, v, w, u, s: Fn.WKV_6STATE.apply(B, T, C, H, r, k, v, w, u, s),
          lambda r, k, v, w, u, s: O.wkv6(r, k, v, w, u, H, s0=s), (r, k, v, wt, uh, s))


def test_host_pipeline_matches_resident_run():
    """Operands in pinned host memory, streamed in batch slices: same bits as the resident run."""
    import rwkv_cuda_b200 as R
    B, T, H, N = 5, 64, 2, 64          # 5 rows in slices of 2: the last slice is ragged
    bf = torch.bfloat16
    inp = Hh.v7_inputs(B, T, H, N, seed=9)
    host_in = {n: inp[n].to(bf).view(B, T, H, N).contiguous().pin_memory() for n in ("r", "w", "k", "v", "a", "b", "dy")}
    host_in.update(s0=inp["s0"].contiguous().pin_memory(), dsT=inp["dsT"].contiguous().pin_memory())
    host_out = {n: torch.empty(B, T, H, N, dtype=bf).pin_memory() for n in R.host_pipeline.Wkv7HostPipeline.OUT}
    host_out.update(sT=torch.empty(B, H, N, N).pin_memory(), ds0=torch.empty(B, H, N, N).pin_memory())
    pipe = R.host_pipeline.Wkv7HostPipeline(T, H, N, DEV, slice_batch=2)
    for _ in range(2):                  # twice: the device buffer sets are reused
        pipe.forward_backward(host_in, host_out)
        pipe.synchronize()
    d = {n: t.to(DEV) for n, t in host_in.items()}
    y, sT, ds0 = torch.empty_like(d["r"]), torch.empty_like(d["s0"]), torch.empty_like(d["s0"])
    s = torch.empty(B, H, T // 16, N, N, device=DEV)
    sa = torch.empty(B, T, H, N, device=DEV)
    R.ops.wkv7_forward(d["s0"], d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], y, sT, s, sa)
    g = [torch.empty_like(y) for _ in range(6)]
    R.ops.wkv7_backward(d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], d["dy"], d["dsT"], s, sa, ds0, *g)
    torch.cuda.synchronize()
    want = dict(y=y, sT=sT, ds0=ds0, **dict(zip(("dr", "dw", "dk", "dv", "da", "db"), g)))
    for n, t in want.items():
        assert torch.equal(host_out[n], t.cpu()), n
