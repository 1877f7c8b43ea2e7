"""`load(...)`: stands in for `torch.utils.cpp_extension.load` in the reference harnesses.

Each reference harness JIT-compiles its kernel with
    load(name=..., sources=[...], extra_cuda_cflags=[... -D_N_=64 ...], [is_python_module=False])
and then calls `<module>.forward/.backward` (pybind modules: wkv, timex, wkv5, wkv5a, wkv6,
wkv6state) or `torch.ops.<name>.forward/.backward` (TORCH_LIBRARY-only modules: the three
rwkv7_* operators).  This shim accepts the same call, ignores `sources`, reads the -D flags
(the reference bakes head size, T, chunk length and dtype into the binary; here they are
runtime values that are checked against the flags), and returns / registers callables with
the reference's argument order that run the prebuilt sm_100a library.
"""
import re
import types

import torch

from . import ops

_PYBIND = {
    "wkv": (ops.wkv4_forward, ops.wkv4_backward),            # wkv/cuda/wkv_op.cpp:13-16
    "timex": (ops.timex_forward, ops.timex_backward),        # depthwise_conv1d/cuda/timex_op.cpp:13-16
    "wkv5": (ops.wkv5_forward, ops.wkv5_backward),           # wkv5_bf16/cuda/wkv5_op.cpp:14-17
    "wkv5a": (ops.wkv5a_forward, ops.wkv5a_backward),        # wkv5a/cuda/wkv5a_op.cpp:18-21
    "wkv6": (ops.wkv6_forward, ops.wkv6_backward),           # wkv6/cuda/wkv6_op.cpp:14-17
    "wkv6state": (ops.wkv6state_forward, ops.wkv6state_backward),  # wkv6_state/cuda/wkv6state_op.cpp:14-17
}

_V7_SCHEMAS = {
    # rwkv7_fast_fused/cuda/rwkv7_clampw.cpp:12,19
    "rwkv7_clampw": (
        "forward(Tensor r, Tensor w, Tensor k, Tensor v, Tensor a, Tensor b, Tensor(a!) y, Tensor(b!) s, Tensor(c!) sa) -> ()",
        "backward(Tensor r, Tensor w, Tensor k, Tensor v, Tensor a, Tensor b, Tensor dy, Tensor s, Tensor sa, "
        "Tensor(a!) dr, Tensor(b!) dw, Tensor(c!) dk, Tensor(d!) dv, Tensor(e!) da, Tensor(f!) db) -> ()"),
    # rwkv7_fast_fused/cuda/rwkv7_state_clampw.cpp:12,19
    "rwkv7_state_clampw": (
        "forward(Tensor s0, Tensor r, Tensor w, Tensor k, Tensor v, Tensor a, Tensor b, Tensor(a!) y, Tensor(b!) s, Tensor(c!) sa) -> ()",
        "backward(Tensor r, Tensor w, Tensor k, Tensor v, Tensor a, Tensor b, Tensor dy, Tensor s, Tensor sa, "
        "Tensor(g!) ds0, Tensor(a!) dr, Tensor(b!) dw, Tensor(c!) dk, Tensor(d!) dv, Tensor(e!) da, Tensor(f!) db) -> ()"),
    # rwkv7_fast_fused/cuda/rwkv7_statepassing_clampw.cpp:12,19
    "rwkv7_statepassing_clampw": (
        "forward(Tensor s0, Tensor r, Tensor w, Tensor k, Tensor v, Tensor a, Tensor b, Tensor(a!) y, Tensor(h!) sT, Tensor(b!) s, Tensor(c!) sa) -> ()",
        "backward(Tensor r, Tensor w, Tensor k, Tensor v, Tensor a, Tensor b, Tensor dy, Tensor dsT, Tensor s, Tensor sa, "
        "Tensor(g!) ds0, Tensor(a!) dr, Tensor(b!) dw, Tensor(c!) dk, Tensor(d!) dv, Tensor(e!) da, Tensor(f!) db) -> ()"),
}

_registered = {}


def parse_defines(flags):
    """{'_N_': 64, '_FP32_': True, ...} from a list of nvcc flags."""
    out = {}
    for f in flags or ():
        for m in re.finditer(r"-D\s*(\w+)(?:=(\S+))?", f):
            val = m.group(2)
            out[m.group(1)] = True if val is None else (int(val) if re.fullmatch(r"-?\d+", val) else val)
    return out


def _v7_impls(name, defs):
    chunk = defs.get("_CHUNK_LEN_")
    head = defs.get("_N_")
    want = torch.float32 if defs.get("_FP32_") else torch.bfloat16

    def check(r, s):
        if r.dtype != want:
            raise TypeError(f"{name}: built for {want} (flag -D_FP32_ {'set' if defs.get('_FP32_') else 'not set'}), got {r.dtype}")
        if head is not None and r.shape[-1] != head:
            raise RuntimeError(f"{name}: built with -D_N_={head}, got head size {r.shape[-1]}")
        if chunk is not None and r.shape[1] % chunk != 0:
            raise RuntimeError(f"{name}: T={r.shape[1]} is not a multiple of -D_CHUNK_LEN_={chunk}")

    if name == "rwkv7_clampw":
        def forward(r, w, k, v, a, b, y, s, sa):
            check(r, s)
            ops.wkv7_forward(None, r, w, k, v, a, b, y, None, s, sa)

        def backward(r, w, k, v, a, b, dy, s, sa, dr, dw, dk, dv, da, db):
            check(r, s)
            ops.wkv7_backward(r, w, k, v, a, b, dy, None, s, sa, None, dr, dw, dk, dv, da, db)
    elif name == "rwkv7_state_clampw":
        def forward(s0, r, w, k, v, a, b, y, s, sa):
            check(r, s)
            ops.wkv7_forward(s0, r, w, k, v, a, b, y, None, s, sa)

        def backward(r, w, k, v, a, b, dy, s, sa, ds0, dr, dw, dk, dv, da, db):
            check(r, s)
            ops.wkv7_backward(r, w, k, v, a, b, dy, None, s, sa, ds0, dr, dw, dk, dv, da, db)
    else:
        def forward(s0, r, w, k, v, a, b, y, sT, s, sa):
            check(r, s)
            ops.wkv7_forward(s0, r, w, k, v, a, b, y, sT, s, sa)

        def backward(r, w, k, v, a, b, dy, dsT, s, sa, ds0, dr, dw, dk, dv, da, db):
            check(r, s)
            ops.wkv7_backward(r, w, k, v, a, b, dy, dsT, s, sa, ds0, dr, dw, dk, dv, da, db)
    return forward, backward


def load(name, sources=None, extra_cflags=None, extra_cuda_cflags=None, is_python_module=True, verbose=False,
         **_ignored):
    """Drop-in for torch.utils.cpp_extension.load for the reference's extension names."""
    defs = parse_defines(extra_cuda_cflags)
    if name in _V7_SCHEMAS:
        fwd, bwd = _v7_impls(name, defs)
        if name not in _registered:
            lib = torch.library.Library(name, "DEF")
            for schema in _V7_SCHEMAS[name]:
                lib.define(schema)
            _registered[name] = {"lib": lib, "forward": fwd, "backward": bwd}
            lib.impl("forward", lambda *a: _registered[name]["forward"](*a), "CUDA")
            lib.impl("backward", lambda *a: _registered[name]["backward"](*a), "CUDA")
        else:  # re-load with other flags (e.g. fp32 after bf16): swap the bound implementation
            _registered[name].update(forward=fwd, backward=bwd)
        mod = types.SimpleNamespace(forward=fwd, backward=bwd, defines=defs, __name__=name)
        return None if not is_python_module else mod
    if name not in _PYBIND:
        raise ValueError(f"load: unknown extension name '{name}' (known: {sorted(_PYBIND) + sorted(_V7_SCHEMAS)})")
    fwd, bwd = _PYBIND[name]
    head = defs.get("_N_", defs.get("N"))

    def forward(*args):
        _check_head(name, head, args)
        return fwd(*args)

    def backward(*args):
        _check_head(name, head, args)
        return bwd(*args)

    return types.SimpleNamespace(forward=forward, backward=backward, defines=defs, __name__=name)


def _check_head(name, head, args):
    # (B, T, C, H, ...) leading ints for the multi-head operators
    if head is not None and name.startswith("wkv") and name != "wkv" and len(args) > 3:
        C, H = args[2], args[3]
        if isinstance(C, int) and isinstance(H, int) and H > 0 and C // H != head:
            raise RuntimeError(f"{name}: built with head size {head}, called with C/H = {C // H}")
