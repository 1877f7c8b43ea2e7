"""CPU tier: the C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments with status codes (no kernel is launched, no GPU is needed)."""
import ctypes
import os

import pytest
import torch

import rwkv_cuda_b200 as R
from rwkv_cuda_b200 import _lib


def test_library_exports_every_declared_symbol():
    protos = _lib.prototypes()
    names = [n for _, n, _ in protos]
    assert len(names) == len(set(names)) and len(names) >= 25
    raw = ctypes.CDLL(_lib.LIBPATH)
    for name in names:
        assert hasattr(raw, name), f"{name} declared in include/rwkvb200.h but not exported"
    for must in ("rwkvb200_wkv7_forward", "rwkvb200_wkv7_backward", "rwkvb200_wkv4_forward", "rwkvb200_timex_backward",
                 "rwkvb200_wkv5_backward", "rwkvb200_wkv5a_forward", "rwkvb200_wkv6_backward",
                 "rwkvb200_wkv6state_backward_ex", "rwkvb200_wkv6_backward_noalloc"):
        assert must in names


def test_identity_and_error_strings():
    L = _lib.lib()
    assert L.rwkvb200_built_for_sm() == 100
    assert L.rwkvb200_version() >= 100
    assert L.rwkvb200_strerror(0) == b"ok"
    assert L.rwkvb200_strerror(-3) == b"misaligned pointer"


def test_status_codes_without_launch():
    L = _lib.lib()
    one = ctypes.c_void_p(16)
    # bad sizes
    assert L.rwkvb200_wkv4_forward(0, 4, 4, one, one, one, one, one, None) == -1
    assert b"must be positive" in L.rwkvb200_last_error()
    # null pointer
    assert L.rwkvb200_wkv4_forward(1, 4, 4, None, one, one, one, one, None) == -2
    assert b"'w'" in L.rwkvb200_last_error()
    # C not a multiple of H, head size too large, unknown dtype
    assert L.rwkvb200_wkv5_forward(1, 1, 4, 10, 3, one, one, one, one, one, one, None) == -1
    assert L.rwkvb200_wkv5_forward(1, 1, 4, 256, 1, one, one, one, one, one, one, None) == -4
    assert L.rwkvb200_wkv6_forward(7, 1, 4, 64, 1, one, one, one, one, one, one, None) == -1
    # RWKV-7: T must be a multiple of chunk_len; s and sa come together
    args7 = [one] * 6
    assert L.rwkvb200_wkv7_forward(1, 1, 20, 1, 64, 16, None, *args7, one, None, one, one, None) == -1
    assert b"multiple of chunk_len" in L.rwkvb200_last_error()
    assert L.rwkvb200_wkv7_forward(1, 1, 32, 1, 64, 16, None, *args7, one, None, one, None, None) == -1
    # misaligned tensor on the tensor-core path
    odd = ctypes.c_void_p(18)
    assert L.rwkvb200_wkv7_forward(1, 1, 32, 1, 64, 16, None, odd, *args7[1:], one, None, one, one, None) == -3
    # path selection is range checked, and the tensor-core path refuses other shapes
    assert L.rwkvb200_wkv7_select_path(7) == -1
    assert L.rwkvb200_wkv7_select_path(2) == 0
    assert L.rwkvb200_wkv7_forward(0, 1, 32, 1, 64, 16, None, *args7, one, None, one, one, None) == -4
    assert L.rwkvb200_wkv7_select_path(0) == 0
    # the allocation-free entry point refuses what does not fit its built-in buffer
    limit = L.rwkvb200_wkv6_backward_noalloc_max_elems()
    assert limit == 8 << 20
    assert L.rwkvb200_wkv6_backward_noalloc(1, 1, limit // 64 + 1, 64, 1, *([one] * 11), None) == -1
    assert b"exceeds the built-in scratch" in L.rwkvb200_last_error()
    assert L.rwkvb200_wkv6_scratch_bytes(2, 3, 4) == 2 * 3 * 4 * 16


def test_ops_refuse_cpu_tensors():
    z = torch.zeros(1, 4, 4)
    with pytest.raises(RuntimeError, match="CUDA device"):
        R.ops.wkv4_forward(1, 4, 4, torch.zeros(4), torch.zeros(4), z, z, z.clone())
    x = torch.zeros(1, 16, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA device"):
        R.ops.wkv7_forward(None, x, x, x, x, x, x, x.clone(), None, None, None)


def test_missing_library_is_loud(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIBPATH", os.path.join(os.path.dirname(_lib.LIBPATH), "does_not_exist.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.lib()
