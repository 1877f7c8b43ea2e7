"""torch.autograd.Function mirrors of the reference harnesses' operators, same class names,
same forward/backward argument order and the same pre/post tensor ops around the kernels.
Module-level globals of the reference (HEAD_SIZE, B, T, C ...) are taken from the tensors.
"""
import torch

from . import ops


class WKV(torch.autograd.Function):
    """RWKV-4 (wkv/run.py:89-117): w -> -exp(w) before, per-batch gw/gu summed after."""

    @staticmethod
    def forward(ctx, B, T, C, w, u, k, v):
        ctx.B, ctx.T, ctx.C = B, T, C
        w = -torch.exp(w.contiguous())
        u, k, v = u.contiguous(), k.contiguous(), v.contiguous()
        ctx.save_for_backward(w, u, k, v)
        y = torch.empty((B, T, C), device=k.device, dtype=torch.float32)
        ops.wkv4_forward(B, T, C, w, u, k, v, y)
        return y

    @staticmethod
    def backward(ctx, gy):
        B, T, C = ctx.B, ctx.T, ctx.C
        w, u, k, v = ctx.saved_tensors
        gw = torch.zeros((B, C), device=k.device)
        gu = torch.zeros((B, C), device=k.device)
        gk = torch.empty((B, T, C), device=k.device)
        gv = torch.empty((B, T, C), device=k.device)
        ops.wkv4_backward(B, T, C, w, u, k, v, gy.contiguous(), gw, gu, gk, gv)
        return None, None, None, gw.sum(dim=0), gu.sum(dim=0), gk, gv


class TimeX(torch.autograd.Function):
    """depthwise_conv1d (depthwise_conv1d/run.py:76-102); gw is reduced over the batch inside the kernel."""

    @staticmethod
    def forward(ctx, w, k, B, C, T, eps):
        ctx.B, ctx.C, ctx.T = B, C, T
        w, k = w.contiguous(), k.contiguous()
        ctx.save_for_backward(w, k)
        wk = torch.empty((B, C, T), device=k.device, dtype=torch.float32)
        ops.timex_forward(w, k, wk, eps, B, C, T)
        return wk

    @staticmethod
    def backward(ctx, gwk):
        w, k = ctx.saved_tensors
        gw = torch.empty((ctx.C, ctx.T), device=k.device, dtype=torch.float32)
        gk = torch.empty((ctx.B, ctx.C, ctx.T), device=k.device, dtype=torch.float32)
        ops.timex_backward_reduced(w, k, gwk.contiguous(), gw, gk, ctx.B, ctx.C, ctx.T)
        return gw, gk, None, None, None, None


class WKV_5(torch.autograd.Function):
    """RWKV-5, bf16 or fp32 (wkv5_bf16/run.py:44-88, wkv5/run.py:469-504)."""

    @staticmethod
    def forward(ctx, B, T, C, H, r, k, v, w, u):
        with torch.no_grad():
            assert r.dtype == k.dtype == v.dtype == w.dtype == u.dtype
            ctx.B, ctx.T, ctx.C, ctx.H = B, T, C, H
            r, k, v, w, u = (x.contiguous() for x in (r, k, v, w, u))
            ew = (-torch.exp(w.float())).contiguous()
            eew = torch.exp(ew).contiguous()
            y = torch.empty((B, T, C), device=r.device, dtype=r.dtype)
            # the chunk-start states are kept for the backward (no second pass over the sequence there)
            saved = torch.empty(ops.wkv5_saved_bytes(B, T, C), dtype=torch.uint8, device=r.device)
            ctx.saved_valid = ops.wkv5_forward_saved(B, T, C, H, r, k, v, eew, u, y, saved)
            ctx.save_for_backward(r, k, v, eew, ew, u, saved)
            return y

    @staticmethod
    def backward(ctx, gy):
        with torch.no_grad():
            B, T, C, H = ctx.B, ctx.T, ctx.C, ctx.H
            r, k, v, eew, ew, u, saved = ctx.saved_tensors
            gr, gk, gv = (torch.empty((B, T, C), device=gy.device, dtype=r.dtype) for _ in range(3))
            gw, gu = (torch.empty((B, C), device=gy.device, dtype=r.dtype) for _ in range(2))
            # the harness sums bf16 (B,C) partials in bf16 (wkv5_bf16/run.py:83-87); here the unrounded fp32
            # partials are summed in fp32 on the device and rounded once
            gw32, gu32 = (torch.empty((B, C), device=gy.device, dtype=torch.float32) for _ in range(2))
            ops.wkv5_backward_saved(B, T, C, H, r, k, v, eew, ew, u, gy.contiguous(), gr, gk, gv, gw, gu, saved,
                                    ctx.saved_valid, gw32, gu32)
            sums = torch.empty((2, C), device=gy.device, dtype=torch.float32)
            ops.reduce_batch_partials(gw32, sums[0])
            ops.reduce_batch_partials(gu32, sums[1])
            shape = u.shape
            return (None, None, None, None, gr, gk, gv, sums[0].to(u.dtype).view(shape), sums[1].to(u.dtype).view(shape))


class WKV_5A(torch.autograd.Function):
    """RWKV-5a (wkv5a/run.py:100-154); r,k,v are (B,T,C), w1,u1,w2,u2 are (H,N)."""

    @staticmethod
    def forward(ctx, r, k, v, w1, u1, w2, u2):
        with torch.no_grad():
            B, T, C = r.shape
            H = w1.shape[0]
            ctx.dims = (B, T, C, H)
            r, k, v, w1, u1, w2, u2 = (x.contiguous() for x in (r, k, v, w1, u1, w2, u2))
            ew1 = (-torch.exp(w1.float())).contiguous()
            eew1 = torch.exp(ew1).contiguous()
            ew2 = (-torch.exp(w2.float())).contiguous()
            eew2 = torch.exp(ew2).contiguous()
            ctx.save_for_backward(r, k, v, eew1, ew1, u1, eew2, ew2, u2)
            y = torch.empty((B, T, C), device=r.device, dtype=r.dtype)
            ops.wkv5a_forward(B, T, C, H, r, k, v, eew1, u1, eew2, u2, y)
            return y

    @staticmethod
    def backward(ctx, gy):
        with torch.no_grad():
            B, T, C, H = ctx.dims
            r, k, v, eew1, ew1, u1, eew2, ew2, u2 = ctx.saved_tensors
            gr, gk, gv = (torch.empty((B, T, C), device=gy.device, dtype=r.dtype) for _ in range(3))
            gw1, gu1, gw2, gu2 = (torch.empty((B, C), device=gy.device, dtype=r.dtype) for _ in range(4))
            ops.wkv5a_backward(B, T, C, H, r, k, v, eew1, ew1, u1, eew2, ew2, u2, gy.contiguous(), gr, gk, gv, gw1,
                               gu1, gw2, gu2)
            return (gr, gk, gv, *(torch.sum(g, 0).view(H, C // H) for g in (gw1, gu1, gw2, gu2)))


class WKV_6(torch.autograd.Function):
    """RWKV-6 (wkv6/run.py:128-170): the kernel receives ew = -exp(w) in fp32."""

    @staticmethod
    def forward(ctx, B, T, C, H, r, k, v, w, u):
        with torch.no_grad():
            ctx.B, ctx.T, ctx.C, ctx.H = B, T, C, H
            r, k, v, w, u = (x.contiguous() for x in (r, k, v, w, u))
            ew = (-torch.exp(w.float())).contiguous()
            ctx.save_for_backward(r, k, v, ew, u)
            y = torch.empty((B, T, C), device=r.device, dtype=r.dtype)
            ops.wkv6_forward(B, T, C, H, r, k, v, ew, u, y)
            return y

    @staticmethod
    def backward(ctx, gy):
        with torch.no_grad():
            B, T, C, H = ctx.B, ctx.T, ctx.C, ctx.H
            r, k, v, ew, u = ctx.saved_tensors
            gr, gk, gv, gw = (torch.empty((B, T, C), device=gy.device, dtype=r.dtype) for _ in range(4))
            gu = torch.empty((B, C), device=gy.device, dtype=r.dtype)
            ops.wkv6_backward(B, T, C, H, r, k, v, ew, u, gy.contiguous(), gr, gk, gv, gw, gu)
            return (None, None, None, None, gr, gk, gv, gw, torch.sum(gu, 0).view(H, C // H))


class WKV_6STATE(torch.autograd.Function):
    """RWKV-6 with initial state (wkv6_state/run.py:80-124): everything in the activation dtype."""

    @staticmethod
    def forward(ctx, B, T, C, H, r, k, v, w, u, s):
        with torch.no_grad():
            ctx.B, ctx.T, ctx.C, ctx.H = B, T, C, H
            r, k, v, w, u, s = (x.contiguous() for x in (r, k, v, w, u, s))
            ctx.save_for_backward(r, k, v, w, u, s)
            y = torch.empty((B, T, C), device=r.device, dtype=r.dtype)
            ops.wkv6state_forward(B, T, C, H, r, k, v, w, u, s, y)
            return y

    @staticmethod
    def backward(ctx, gy):
        with torch.no_grad():
            B, T, C, H = ctx.B, ctx.T, ctx.C, ctx.H
            r, k, v, w, u, s = ctx.saved_tensors
            gr, gk, gv, gw = (torch.empty((B, T, C), device=gy.device, dtype=r.dtype) for _ in range(4))
            gu = torch.empty((B, C), device=gy.device, dtype=r.dtype)
            gs = torch.empty((B, H, C // H, C // H), device=gy.device, dtype=r.dtype)
            ops.wkv6state_backward(B, T, C, H, r, k, v, w, u, s, gy.contiguous(), gr, gk, gv, gw, gu, gs)
            return (None, None, None, None, gr, gk, gv, gw, torch.sum(gu, 0).view(H, C // H), gs)


class WKV_6STATE_EX(torch.autograd.Function):
    """RWKV-6 with fp32 state in and out (state passing); no counterpart class in the reference."""

    @staticmethod
    def forward(ctx, r, k, v, w, u, s0):
        with torch.no_grad():
            B, T, C = r.shape
            H = u.shape[0]
            ctx.dims = (B, T, C, H)
            r, k, v, w, u, s0 = (x.contiguous() for x in (r, k, v, w, u, s0))
            y = torch.empty((B, T, C), device=r.device, dtype=r.dtype)
            sT = torch.empty_like(s0)
            # the chunk-start states are kept for the backward (half the size of its scratch buffer is used)
            saved = torch.empty(ops.wkv6_saved_bytes(B, T, C), dtype=torch.uint8, device=r.device)
            ctx.saved_valid = ops.wkv6state_forward_saved(B, T, C, H, r, k, v, w, u, s0, y, sT, saved)
            ctx.save_for_backward(r, k, v, w, u, s0, saved)
            return y, sT

    @staticmethod
    def backward(ctx, gy, dsT):
        with torch.no_grad():
            B, T, C, H = ctx.dims
            r, k, v, w, u, s0, saved = ctx.saved_tensors
            gr, gk, gv, gw = (torch.empty((B, T, C), device=gy.device, dtype=r.dtype) for _ in range(4))
            gu = torch.empty((B, C), device=gy.device, dtype=r.dtype)
            ds0 = torch.empty_like(s0)
            ops.wkv6state_backward_saved(B, T, C, H, r, k, v, w, u, s0, gy.contiguous(), dsT.contiguous(), gr, gk, gv,
                                         gw, gu, ds0, saved, ctx.saved_valid)
            return gr, gk, gv, gw, torch.sum(gu.float(), 0).view(H, C // H).to(u.dtype), ds0


CHUNK_LEN = 16


def _v7_saved(r):
    B, T, H, N = r.shape
    s = torch.empty(B, H, T // CHUNK_LEN, N, N, dtype=torch.float32, device=r.device)
    sa = torch.empty(B, T, H, N, dtype=torch.float32, device=r.device)
    return s, sa


def _v7_check(*xs):
    r = xs[0]
    assert r.shape[1] % CHUNK_LEN == 0
    assert all(i.dtype == r.dtype for i in xs)
    assert all(i.is_contiguous() for i in xs)


class RWKV7_CLAMPW_CUDA_OP(torch.autograd.Function):
    """rwkv7_fast_fused/rwkv7_cuda_benchmark.py:76-96; inputs (B,T,H,N)."""

    @staticmethod
    def forward(ctx, r, w, k, v, a, b):
        _v7_check(r, w, k, v, a, b)
        y = torch.empty_like(v)
        s, sa = _v7_saved(r)
        ops.wkv7_forward(None, r, w, k, v, a, b, y, None, s, sa)
        ctx.save_for_backward(r, w, k, v, a, b, s, sa)
        return y

    @staticmethod
    def backward(ctx, dy):
        r, w, k, v, a, b, s, sa = ctx.saved_tensors
        dr, dw, dk, dv, da, db = (torch.empty_like(x) for x in (r, w, k, v, a, b))
        ops.wkv7_backward(r, w, k, v, a, b, dy.contiguous(), None, s, sa, None, dr, dw, dk, dv, da, db)
        return dr, dw, dk, dv, da, db


class RWKV7_STATE_CLAMPW_CUDA_OP(torch.autograd.Function):
    """rwkv7_fast_fused/rwkv7_cuda_benchmark_state.py:75-99."""

    @staticmethod
    def forward(ctx, s0, r, w, k, v, a, b):
        _v7_check(r, w, k, v, a, b)
        assert s0.dtype == torch.float and s0.is_contiguous()
        y = torch.empty_like(v)
        s, sa = _v7_saved(r)
        ops.wkv7_forward(s0, r, w, k, v, a, b, y, None, s, sa)
        ctx.save_for_backward(r, w, k, v, a, b, s, sa)
        return y

    @staticmethod
    def backward(ctx, dy):
        r, w, k, v, a, b, s, sa = ctx.saved_tensors
        B, T, H, N = r.shape
        dr, dw, dk, dv, da, db = (torch.empty_like(x) for x in (r, w, k, v, a, b))
        ds0 = torch.empty(B, H, N, N, dtype=torch.float32, device=r.device)
        ops.wkv7_backward(r, w, k, v, a, b, dy.contiguous(), None, s, sa, ds0, dr, dw, dk, dv, da, db)
        return ds0, dr, dw, dk, dv, da, db


class RWKV7_STATE_PASSING_CLAMPW_CUDA_OP(torch.autograd.Function):
    """rwkv7_fast_fused/rwkv7_cuda_benchmark_state_passing.py:75-99: returns (y, sT)."""

    @staticmethod
    def forward(ctx, s0, r, w, k, v, a, b):
        B, T, H, N = r.shape
        _v7_check(r, w, k, v, a, b)
        assert s0.dtype == torch.float and s0.is_contiguous()
        y = torch.empty_like(v)
        sT = torch.empty_like(s0)
        s, sa = _v7_saved(r)
        ops.wkv7_forward(s0, r, w, k, v, a, b, y, sT, s, sa)
        ctx.save_for_backward(r, w, k, v, a, b, s, sa)
        return y.view(B, T, H * N), sT

    @staticmethod
    def backward(ctx, dy, dsT):
        r, w, k, v, a, b, s, sa = ctx.saved_tensors
        assert dsT.dtype == torch.float
        ds0 = torch.empty_like(dsT)
        dr, dw, dk, dv, da, db = (torch.empty_like(x) for x in (r, w, k, v, a, b))
        ops.wkv7_backward(r, w, k, v, a, b, dy.contiguous(), dsT.contiguous(), s, sa, ds0, dr, dw, dk, dv, da, db)
        return ds0, dr, dw, dk, dv, da, db


def _heads(x, head_size):
    B, T, HC = x.shape
    return x.view(B, T, HC // head_size, head_size)


def RWKV7_CLAMPW_CUDA(r, w, k, v, a, b, head_size=64):
    B, T, HC = r.shape
    return RWKV7_CLAMPW_CUDA_OP.apply(*(_heads(i, head_size) for i in (r, w, k, v, a, b))).view(B, T, HC)


def RWKV7_STATE_CLAMPW_CUDA(s0, r, w, k, v, a, b):
    B, T, HC = r.shape
    return RWKV7_STATE_CLAMPW_CUDA_OP.apply(s0, *(_heads(i, s0.shape[-1]) for i in (r, w, k, v, a, b))).view(B, T, HC)


def RWKV7_STATE_PASSING_CLAMPW_CUDA(s0, r, w, k, v, a, b):
    return RWKV7_STATE_PASSING_CLAMPW_CUDA_OP.apply(s0, *(_heads(i, s0.shape[-1]) for i in (r, w, k, v, a, b)))
