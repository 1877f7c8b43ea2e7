"""Tensor-level wrappers of the C ABI: same argument order as the reference bindings
(`forward(...)` / `backward(...)` of each *_op.cpp), outputs written in place, returning None.

Tensors must live on a CUDA device and be contiguous; pointers, sizes and the current stream
are handed to librwkvb200.so.  PyTorch is used for memory and streams only.
"""
import torch

from . import _lib
from ._lib import BF16, F32, call

_scratch = {}


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _dev(t, name="tensor"):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name}: tensor must be on a CUDA device (there is no CPU path)")
    return torch.cuda.device(t.device)


def _ptr(t, name, dtype=None):
    if t is None:
        return None
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name}: expected a tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise RuntimeError(f"{name}: tensor must be on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name}: expected {dtype}, got {t.dtype}")
    return t.data_ptr()


def _dt(t, name):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"{name}: dtype {t.dtype} not supported (float32 or bfloat16)")


def _ptrs(dtype, **tensors):
    return [_ptr(t, n, dtype) for n, t in tensors.items()]


def _numel(t, n, name):
    if t.numel() != n:
        raise RuntimeError(f"{name}: expected {n} elements, got {tuple(t.shape)}")


def scratch(nbytes, device):
    """Per-device, per-stream scratch buffer that grows on demand (used by the wkv6 backward)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def free_scratch(device=None):
    """Drops the cached scratch buffers (of one device, or of all): they grow to the largest request seen per
    (device, stream) and are otherwise kept for the life of the process.  Call it with no work of this library
    in flight on those streams."""
    for key in [k for k in _scratch if device is None or k[0] == torch.device(device).index]:
        del _scratch[key]


# ---- RWKV-4 (wkv/cuda/wkv_op.cpp:6-11) ------------------------------------------------
def wkv4_forward(B, T, C, w, u, k, v, y):
    f = torch.float32
    for t, n, name in ((w, C, "w"), (u, C, "u"), (k, B * T * C, "k"), (v, B * T * C, "v"), (y, B * T * C, "y")):
        _numel(t, n, name)
    with _dev(k, "k"):
        call("rwkvb200_wkv4_forward", B, T, C, *_ptrs(f, w=w, u=u, k=k, v=v, y=y), _stream(k))


def wkv4_backward(B, T, C, w, u, k, v, gy, gw, gu, gk, gv):
    f = torch.float32
    for t, n, name in ((w, C, "w"), (u, C, "u"), (k, B * T * C, "k"), (v, B * T * C, "v"), (gy, B * T * C, "gy"),
                       (gw, B * C, "gw"), (gu, B * C, "gu"), (gk, B * T * C, "gk"), (gv, B * T * C, "gv")):
        _numel(t, n, name)
    with _dev(k, "k"):
        call("rwkvb200_wkv4_backward", B, T, C, *_ptrs(f, w=w, u=u, k=k, v=v, gy=gy, gw=gw, gu=gu, gk=gk, gv=gv),
             _stream(k))


# ---- depthwise_conv1d (depthwise_conv1d/cuda/timex_op.cpp:6-11) -----------------------
def timex_forward(w, k, x, eps, B, C, T):
    f = torch.float32
    for t, n, name in ((w, C * T, "w"), (k, B * C * T, "k"), (x, B * C * T, "x")):
        _numel(t, n, name)
    with _dev(k, "k"):
        call("rwkvb200_timex_forward", *_ptrs(f, w=w, k=k, x=x), float(eps), B, C, T, _stream(k))


def timex_backward(w, k, gwk, gw, gk, B, C, T):
    f = torch.float32
    for t, n, name in ((w, C * T, "w"), (k, B * C * T, "k"), (gwk, B * C * T, "gwk"), (gw, B * C * T, "gw"),
                       (gk, B * C * T, "gk")):
        _numel(t, n, name)
    with _dev(k, "k"):
        call("rwkvb200_timex_backward", *_ptrs(f, w=w, k=k, gwk=gwk, gw=gw, gk=gk), B, C, T, _stream(k))


def timex_backward_reduced(w, k, gwk, gw_sum, gk, B, C, T):
    f = torch.float32
    for t, n, name in ((w, C * T, "w"), (k, B * C * T, "k"), (gwk, B * C * T, "gwk"), (gw_sum, C * T, "gw_sum"),
                       (gk, B * C * T, "gk")):
        _numel(t, n, name)
    with _dev(k, "k"):
        call("rwkvb200_timex_backward_reduced", *_ptrs(f, w=w, k=k, gwk=gwk, gw_sum=gw_sum, gk=gk), B, C, T,
             _stream(k))


# ---- RWKV-5 (wkv5_bf16/cuda/wkv5_op.cpp:8-13, wkv5/cuda/wkv5_op.cpp:6-11) --------------
def wkv5_forward(B, T, C, H, r, k, v, w, u, y):
    d = r.dtype
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w, C, "w"), (u, C, "u"),
                       (y, B * T * C, "y")):
        _numel(t, n, name)
    with _dev(r, "r"):
        call("rwkvb200_wkv5_forward", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v), _ptr(w, "w", torch.float32),
             _ptr(u, "u", d), _ptr(y, "y", d), _stream(r))


def wkv5_backward(B, T, C, H, r, k, v, w, ww, u, gy, gr, gk, gv, gw, gu, gw32=None, gu32=None):
    """gw32, gu32 (optional, both or none): fp32 (B,C) tensors that receive the unrounded partials of gw and gu
    (reduce them with reduce_batch_partials: no bf16 round trip on the parameter gradients)."""
    d = r.dtype
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w, C, "w"), (ww, C, "ww"),
                       (u, C, "u"), (gy, B * T * C, "gy"), (gr, B * T * C, "gr"), (gk, B * T * C, "gk"),
                       (gv, B * T * C, "gv"), (gw, B * C, "gw"), (gu, B * C, "gu")):
        _numel(t, n, name)
    with _dev(r, "r"):
        sc = scratch(_lib.lib().rwkvb200_wkv5_scratch_bytes(B, T, C), r.device)
        if gw32 is None and gu32 is None:
            call("rwkvb200_wkv5_backward_ws", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v),
                 _ptr(w, "w", torch.float32), _ptr(ww, "ww", torch.float32),
                 *_ptrs(d, u=u, gy=gy, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu), sc.data_ptr(), _stream(r))
        else:
            _numel(gw32, B * C, "gw32")
            _numel(gu32, B * C, "gu32")
            call("rwkvb200_wkv5_backward_ws32", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v),
                 _ptr(w, "w", torch.float32), _ptr(ww, "ww", torch.float32),
                 *_ptrs(d, u=u, gy=gy, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu), _ptr(gw32, "gw32", torch.float32),
                 _ptr(gu32, "gu32", torch.float32), sc.data_ptr(), _stream(r))


def wkv5_saved_bytes(B, T, C):
    return _lib.lib().rwkvb200_wkv5_scratch_bytes(B, T, C)


def wkv5_forward_saved(B, T, C, H, r, k, v, w, u, y, saved):
    """Forward that also leaves the chunk-start states in `saved` (uint8 tensor of wkv5_saved_bytes(B,T,C) bytes) for
    wkv5_backward_saved; returns True when they were saved (pass it on as `valid`)."""
    d = r.dtype
    with _dev(r, "r"):
        L = _lib.lib()
        rc = L.rwkvb200_wkv5_forward_saved(_dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v), _ptr(w, "w", torch.float32),
                                           _ptr(u, "u", d), _ptr(y, "y", d), saved.data_ptr(), _stream(r))
        if rc < 0:
            raise _lib.RwkvB200Error(f"rwkvb200_wkv5_forward_saved: {L.rwkvb200_strerror(rc).decode()} ({rc}): "
                                     f"{L.rwkvb200_last_error().decode()}")
        return rc == 0


def wkv5_backward_saved(B, T, C, H, r, k, v, w, ww, u, gy, gr, gk, gv, gw, gu, saved, valid, gw32=None, gu32=None):
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        call("rwkvb200_wkv5_backward_saved", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v),
             _ptr(w, "w", f), _ptr(ww, "ww", f), *_ptrs(d, u=u, gy=gy, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu),
             _ptr(gw32, "gw32", f), _ptr(gu32, "gu32", f), saved.data_ptr(), 1 if valid else 0, _stream(r))


def reduce_batch_partials(partial, out):
    """out (n,) fp32 <- sum over dim 0 of partial (B, n) (bf16 or fp32), accumulated in fp32."""
    B = partial.shape[0]
    n = partial.numel() // B
    _numel(out, n, "out")
    with _dev(partial, "partial"):
        call("rwkvb200_reduce_batch_partials", _dt(partial, "partial"), B, n, _ptr(partial, "partial", partial.dtype),
             _ptr(out, "out", torch.float32), _stream(partial))


# ---- RWKV-5a (wkv5a/cuda/wkv5a_op.cpp:9-17) -------------------------------------------
def wkv5a_forward(B, T, C, H, r, k, v, w1, u1, w2, u2, y):
    d, f = r.dtype, torch.float32
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w1, C, "w1"), (u1, C, "u1"),
                       (w2, C, "w2"), (u2, C, "u2"), (y, B * T * C, "y")):
        _numel(t, n, name)
    with _dev(r, "r"):
        call("rwkvb200_wkv5a_forward", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v), _ptr(w1, "w1", f),
             _ptr(u1, "u1", d), _ptr(w2, "w2", f), _ptr(u2, "u2", d), _ptr(y, "y", d), _stream(r))


def wkv5a_backward(B, T, C, H, r, k, v, w1, ww1, u1, w2, ww2, u2, gy, gr, gk, gv, gw1, gu1, gw2, gu2):
    d, f = r.dtype, torch.float32
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (gy, B * T * C, "gy"),
                       (gr, B * T * C, "gr"), (gk, B * T * C, "gk"), (gv, B * T * C, "gv"), (w1, C, "w1"),
                       (ww1, C, "ww1"), (u1, C, "u1"), (w2, C, "w2"), (ww2, C, "ww2"), (u2, C, "u2"),
                       (gw1, B * C, "gw1"), (gu1, B * C, "gu1"), (gw2, B * C, "gw2"), (gu2, B * C, "gu2")):
        _numel(t, n, name)
    with _dev(r, "r"):
        call("rwkvb200_wkv5a_backward", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v), _ptr(w1, "w1", f),
             _ptr(ww1, "ww1", f), _ptr(u1, "u1", d), _ptr(w2, "w2", f), _ptr(ww2, "ww2", f), _ptr(u2, "u2", d),
             *_ptrs(d, gy=gy, gr=gr, gk=gk, gv=gv, gw1=gw1, gu1=gu1, gw2=gw2, gu2=gu2), _stream(r))


# ---- RWKV-6 (wkv6/cuda/wkv6_op.cpp:8-13) ----------------------------------------------
def wkv6_forward(B, T, C, H, r, k, v, w, u, y):
    d = r.dtype
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w, B * T * C, "w"),
                       (u, C, "u"), (y, B * T * C, "y")):
        _numel(t, n, name)
    with _dev(r, "r"):
        call("rwkvb200_wkv6_forward", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v), _ptr(w, "w", torch.float32),
             _ptr(u, "u", d), _ptr(y, "y", d), _stream(r))


def wkv6_backward(B, T, C, H, r, k, v, w, u, gy, gr, gk, gv, gw, gu):
    d = r.dtype
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w, B * T * C, "w"),
                       (u, C, "u"), (gy, B * T * C, "gy"), (gr, B * T * C, "gr"), (gk, B * T * C, "gk"),
                       (gv, B * T * C, "gv"), (gw, B * T * C, "gw"), (gu, B * C, "gu")):
        _numel(t, n, name)
    with _dev(r, "r"):
        sc = scratch(_lib.lib().rwkvb200_wkv6_scratch_bytes(B, T, C), r.device)
        call("rwkvb200_wkv6_backward", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v),
             _ptr(w, "w", torch.float32), *_ptrs(d, u=u, gy=gy, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu), sc.data_ptr(),
             _stream(r))


def wkv6_backward_noalloc(B, T, C, H, r, k, v, w, u, gy, gr, gk, gv, gw, gu):
    """wkv6_backward for callers that must not allocate: no scratch tensor is created here, the
    library uses its built-in 32 MiB buffer (B*T*C <= 8 Mi elements, else RwkvB200Error).  Calls
    that could overlap on the GPU must be serialised by the caller: they share that buffer."""
    d = r.dtype
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w, B * T * C, "w"),
                       (u, C, "u"), (gy, B * T * C, "gy"), (gr, B * T * C, "gr"), (gk, B * T * C, "gk"),
                       (gv, B * T * C, "gv"), (gw, B * T * C, "gw"), (gu, B * C, "gu")):
        _numel(t, n, name)
    with _dev(r, "r"):
        call("rwkvb200_wkv6_backward_noalloc", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v),
             _ptr(w, "w", torch.float32), *_ptrs(d, u=u, gy=gy, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu), _stream(r))


# ---- RWKV-6 with state (wkv6_state/cuda/wkv6state_op.cpp:8-13) ------------------------
def wkv6state_forward(B, T, C, H, r, k, v, w, u, s, y):
    d = r.dtype
    N = C // H
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w, B * T * C, "w"),
                       (u, C, "u"), (s, B * H * N * N, "s"), (y, B * T * C, "y")):
        _numel(t, n, name)
    with _dev(r, "r"):
        call("rwkvb200_wkv6state_forward", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v, w=w, u=u, s=s, y=y),
             _stream(r))


def wkv6state_backward(B, T, C, H, r, k, v, w, u, s, gy, gr, gk, gv, gw, gu, gs):
    d = r.dtype
    N = C // H
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w, B * T * C, "w"),
                       (u, C, "u"), (s, B * H * N * N, "s"), (gy, B * T * C, "gy"), (gr, B * T * C, "gr"),
                       (gk, B * T * C, "gk"), (gv, B * T * C, "gv"), (gw, B * T * C, "gw"), (gu, B * C, "gu"),
                       (gs, B * H * N * N, "gs")):
        _numel(t, n, name)
    with _dev(r, "r"):
        sc = scratch(_lib.lib().rwkvb200_wkv6_scratch_bytes(B, T, C), r.device)
        call("rwkvb200_wkv6state_backward", _dt(r, "r"), B, T, C, H,
             *_ptrs(d, r=r, k=k, v=v, w=w, u=u, s=s, gy=gy, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu, gs=gs),
             sc.data_ptr(), _stream(r))


def wkv6state_forward_ex(B, T, C, H, r, k, v, w, u, s0, y, sT):
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        call("rwkvb200_wkv6state_forward_ex", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v, w=w, u=u),
             _ptr(s0, "s0", f), _ptr(y, "y", d), _ptr(sT, "sT", f), _stream(r))


def wkv6state_forward_saved(B, T, C, H, r, k, v, w, u, s0, y, sT, saved):
    """Forward that also leaves the chunk-start states in `saved` (uint8 tensor of wkv6_saved_bytes(B,T,C) bytes) for
    wkv6state_backward_saved; returns True when they were saved (pass it on as `valid`)."""
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        rc = _lib.lib().rwkvb200_wkv6state_forward_saved(_dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v, w=w, u=u),
                                                         _ptr(s0, "s0", f), _ptr(y, "y", d), _ptr(sT, "sT", f),
                                                         saved.data_ptr(), _stream(r))
        if rc < 0:
            L = _lib.lib()
            raise _lib.RwkvB200Error(f"rwkvb200_wkv6state_forward_saved: {L.rwkvb200_strerror(rc).decode()} ({rc}): "
                                     f"{L.rwkvb200_last_error().decode()}")
        return rc == 0


def wkv6state_backward_saved(B, T, C, H, r, k, v, w, u, s0, gy, dsT, gr, gk, gv, gw, gu, ds0, saved, valid):
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        call("rwkvb200_wkv6state_backward_saved", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v, w=w, u=u),
             _ptr(s0, "s0", f), _ptr(gy, "gy", d), _ptr(dsT, "dsT", f),
             *_ptrs(d, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu), _ptr(ds0, "ds0", f), saved.data_ptr(), 1 if valid else 0, _stream(r))


def wkv6_saved_bytes(B, T, C):
    return _lib.lib().rwkvb200_wkv6_scratch_bytes(B, T, C)


def tsplit_segments(B, T, H, device):
    """How many time segments the split forward should use for this launch: 1 unless the launch has at most a
    quarter as many (batch, head) units as the GPU has SMs (the unsplit tcgen05 forward walks a unit's chunks at
    about 2.5 k cycles per 32 tokens, which a split only beats with many idle SMs); then one segment per idle SM,
    at least 512 tokens each, whole 16-token chunks.  Measured, RWKV-6 with state, one sequence of 8 heads:
    T 16384 0.61 ms unsplit, 0.29 ms in 16 segments; T 65536 2.43 -> 0.73 ms; 64 heads: the split loses."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    units = max(1, B * H)
    if units * 4 > sms:
        return 1
    k = max(1, min(sms // units, T // 512))
    while k > 1 and (T % k != 0 or (T // k) % 16 != 0):
        k -= 1
    return k


def wkv5_forward_tsplit(B, T, C, H, r, k, v, w, u, y, segments=None):
    """RWKV-5 forward split over time (few (batch, head) units: the segments run at the same time)."""
    d = r.dtype
    for t, n, name in ((r, B * T * C, "r"), (k, B * T * C, "k"), (v, B * T * C, "v"), (w, C, "w"), (u, C, "u"),
                       (y, B * T * C, "y")):
        _numel(t, n, name)
    with _dev(r, "r"):
        K = segments or tsplit_segments(B, T, H, r.device)
        wk = scratch(_lib.lib().rwkvb200_wkv6_tsplit_bytes(B, T, C, H, K), r.device)
        call("rwkvb200_wkv5_forward_tsplit", _dt(r, "r"), B, T, C, H, K, *_ptrs(d, r=r, k=k, v=v),
             _ptr(w, "w", torch.float32), _ptr(u, "u", d), _ptr(y, "y", d), wk.data_ptr(), _stream(r))


def wkv6state_forward_tsplit(B, T, C, H, r, k, v, w, u, s0, y, sT, segments=None):
    """RWKV-6 forward with fp32 state in / out, split over time."""
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        K = segments or tsplit_segments(B, T, H, r.device)
        wk = scratch(_lib.lib().rwkvb200_wkv6_tsplit_bytes(B, T, C, H, K), r.device)
        call("rwkvb200_wkv6state_forward_tsplit", _dt(r, "r"), B, T, C, H, K, *_ptrs(d, r=r, k=k, v=v, w=w, u=u),
             _ptr(s0, "s0", f), _ptr(y, "y", d), _ptr(sT, "sT", f), wk.data_ptr(), _stream(r))


def wkv6state_backward_ex(B, T, C, H, r, k, v, w, u, s0, gy, dsT, gr, gk, gv, gw, gu, ds0):
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        sc = scratch(_lib.lib().rwkvb200_wkv6_scratch_bytes(B, T, C), r.device)
        call("rwkvb200_wkv6state_backward_ex", _dt(r, "r"), B, T, C, H, *_ptrs(d, r=r, k=k, v=v, w=w, u=u),
             _ptr(s0, "s0", f), _ptr(gy, "gy", d), _ptr(dsT, "dsT", f),
             *_ptrs(d, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu), _ptr(ds0, "ds0", f), sc.data_ptr(), _stream(r))


# ---- RWKV-7 (rwkv7_fast_fused/cuda/rwkv7_*clampw.cpp:12-24) ----------------------------
def _v7_dims(r, s):
    if r.dim() != 4:
        raise RuntimeError(f"r: expected (B,T,H,N), got {tuple(r.shape)}")
    B, T, H, N = r.shape
    if s is None:
        return B, T, H, N, 16
    n_chunks = s.numel() // (B * H * N * N)
    if n_chunks <= 0 or s.numel() != B * H * n_chunks * N * N or T % n_chunks != 0:
        raise RuntimeError(f"s: shape {tuple(s.shape)} is not (B,H,T/chunk_len,N,N) for r {tuple(r.shape)}")
    return B, T, H, N, T // n_chunks


def wkv7_forward(s0, r, w, k, v, a, b, y, sT, s, sa):
    """All three reference operators: s0 / sT may be None (zero initial state / no final state)."""
    B, T, H, N, chunk = _v7_dims(r, s)
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        call("rwkvb200_wkv7_forward", _dt(r, "r"), B, T, H, N, chunk, _ptr(s0, "s0", f),
             *_ptrs(d, r=r, w=w, k=k, v=v, a=a, b=b, y=y), _ptr(sT, "sT", f), _ptr(s, "s", f), _ptr(sa, "sa", f),
             _stream(r))


def wkv7_state_update(state, r, w, k, v, a, b, y):
    """Inference: advance `state` (B,H,N,N fp32) in place by the T tokens of r..b (B,T,H,N) and write y."""
    B, T, H, N = r.shape
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        call("rwkvb200_wkv7_state_update", _dt(r, "r"), B, T, H, N, _ptr(state, "state", f),
             *_ptrs(d, r=r, w=w, k=k, v=v, a=a, b=b, y=y), _stream(r))


def wkv7_backward(r, w, k, v, a, b, dy, dsT, s, sa, ds0, dr, dw, dk, dv, da, db):
    B, T, H, N, chunk = _v7_dims(r, s)
    d, f = r.dtype, torch.float32
    with _dev(r, "r"):
        call("rwkvb200_wkv7_backward", _dt(r, "r"), B, T, H, N, chunk, *_ptrs(d, r=r, w=w, k=k, v=v, a=a, b=b, dy=dy),
             _ptr(dsT, "dsT", f), _ptr(s, "s", f), _ptr(sa, "sa", f), _ptr(ds0, "ds0", f),
             *_ptrs(d, dr=dr, dw=dw, dk=dk, dv=dv, da=da, db=db), _stream(r))
