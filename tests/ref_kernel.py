"""The reference project's own RWKV-7 state-passing CUDA kernel (bf16, N=64, chunk 16), built
for sm_100 by oracle/build_ref.py, callable on torch tensors.  Test infrastructure: used to
check that the library's error against the fp64 oracle is no worse than the reference
kernel's, and (run as a script) to time the reference kernel on the same GPU.

    python tests/ref_kernel.py [B T H]     # prints one JSON line of timings for both kernels
"""
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "_ref", "librwkv7_ref.so")
_lib = None


def available():
    return os.path.exists(LIB)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB)
        vp, i = ctypes.c_void_p, ctypes.c_int
        _lib.ref_rwkv7_sp_forward.argtypes = [i, i, i] + [vp] * 11
        _lib.ref_rwkv7_sp_forward.restype = None
        _lib.ref_rwkv7_sp_backward.argtypes = [i, i, i] + [vp] * 17
        _lib.ref_rwkv7_sp_backward.restype = None
    return _lib


def forward(s0, r, w, k, v, a, b, y, sT, s, sa):
    """Runs on the legacy default stream, as the reference does."""
    B, T, H, N = r.shape
    assert N == 64 and T % 16 == 0 and r.dtype == torch.bfloat16
    torch.cuda.current_stream().synchronize()
    lib().ref_rwkv7_sp_forward(B, T, H, *(t.data_ptr() for t in (s0, r, w, k, v, a, b, y, sT, s, sa)))


def backward(r, w, k, v, a, b, dy, dsT, s, sa, ds0, dr, dw, dk, dv, da, db):
    B, T, H, N = r.shape
    torch.cuda.current_stream().synchronize()
    lib().ref_rwkv7_sp_backward(B, T, H, *(t.data_ptr() for t in (r, w, k, v, a, b, dy, dsT, s, sa, ds0, dr, dw, dk,
                                                                   dv, da, db)))


_other = {}


def other_lib(name):
    """oracle/_ref/lib<name>_ref.so (rwkv5, rwkv6state) or None when it was not built."""
    if name not in _other:
        path = os.path.join(ROOT, "oracle", "_ref", f"lib{name}_ref.so")
        _other[name] = ctypes.CDLL(path) if os.path.exists(path) else None
        L = _other[name]
        if L is not None:
            vp, i = ctypes.c_void_p, ctypes.c_int
            if name == "rwkv5":
                L.ref_wkv5_forward.argtypes = [i] * 4 + [vp] * 6
                L.ref_wkv5_backward.argtypes = [i] * 4 + [vp] * 12
                L.ref_wkv5_forward.restype = L.ref_wkv5_backward.restype = None
            else:
                L.ref_wkv6state_forward.argtypes = [i] * 4 + [vp] * 7
                L.ref_wkv6state_backward.argtypes = [i] * 4 + [vp] * 13
                L.ref_wkv6state_forward.restype = L.ref_wkv6state_backward.restype = None
                L.ref_wkv6state_T.restype = i
    return _other[name]


def run(inp, H, fwd, bwd):
    """inp: dict of CPU fp32 tensors (tests.helpers.v7_inputs).  Returns outputs as a dict."""
    dev = "cuda"
    bf = torch.bfloat16
    B, T, C = inp["r"].shape
    N = C // H
    d = {n: inp[n].to(bf).to(dev).view(B, T, H, N).contiguous() for n in ("r", "w", "k", "v", "a", "b", "dy")}
    s0, dsT = inp["s0"].float().to(dev), inp["dsT"].float().to(dev)
    y = torch.empty(B, T, H, N, dtype=bf, device=dev)
    sT, ds0 = torch.empty_like(s0), torch.empty_like(s0)
    s = torch.empty(B, H, T // 16, N, N, device=dev)
    sa = torch.empty(B, T, H, N, device=dev)
    fwd(s0, d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], y, sT, s, sa)
    g = [torch.empty_like(y) for _ in range(6)]
    bwd(d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], d["dy"], dsT, s, sa, ds0, *g)
    torch.cuda.synchronize()
    return dict(y=y, sT=sT, ds0=ds0, **dict(zip(("dr", "dw", "dk", "dv", "da", "db"), g)))


def _time(fn, n=5):
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = 1e30
    for _ in range(n):
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


if __name__ == "__main__":
    sys.path.insert(0, ROOT)
    import rwkv_cuda_b200 as R
    B, T, H = (int(x) for x in sys.argv[1:4]) if len(sys.argv) >= 4 else (16, 4096, 64)
    N, dev, bf = 64, "cuda", torch.bfloat16
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    mk = lambda sc=1.0: (torch.randn(B, T, H, N, device=dev, generator=g) * sc)
    r, k, v, w = mk(.5).to(bf), mk(.5).to(bf), mk(.5).to(bf), mk().to(bf)
    kk = torch.nn.functional.normalize(mk(), dim=-1)
    a, b, dy = (-kk).to(bf), (kk * torch.sigmoid(mk())).to(bf), mk().to(bf)
    s0, dsT = 0.1 * torch.randn(B, H, N, N, device=dev), torch.randn(B, H, N, N, device=dev)
    y, sT, ds0 = torch.empty_like(r), torch.empty_like(s0), torch.empty_like(s0)
    s, sa = torch.empty(B, H, T // 16, N, N, device=dev), torch.empty(B, T, H, N, device=dev)
    gr = [torch.empty_like(r) for _ in range(6)]
    out = {"shape": [B, T, H, N]}
    for name, f, bw in (("reference_kernel", forward, backward), ("library", R.ops.wkv7_forward, R.ops.wkv7_backward)):
        if name == "reference_kernel" and not available():
            continue
        tf = _time(lambda: f(s0, r, w, k, v, a, b, y, sT, s, sa))
        tb = _time(lambda: bw(r, w, k, v, a, b, dy, dsT, s, sa, ds0, *gr))
        out[name] = {"fwd_ms": tf, "bwd_ms": tb, "tokens_per_s": B * T / ((tf + tb) * 1e-3)}
    print(json.dumps(out))
