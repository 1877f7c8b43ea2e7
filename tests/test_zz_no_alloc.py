"""The allocation-free RWKV-6 backward entry point (collected last on purpose).

Some users of the library run the backward where device memory cannot be allocated (a
latency-critical thread that may not enter the allocator, a runtime that owns all device memory
and hands out fixed buffers, a memory pool that is already fully committed).  rwkvb200_wkv6_backward_noalloc serves them from a fixed buffer inside the library.
It must give the same result as the normal entry point, call after call, and refuse problems
larger than its buffer.
"""
import pytest
import torch

from tests import helpers as Hh

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(dtype, B, T, H, N, seed):
    g = Hh.gen(seed)
    C = H * N
    r, k, v = (0.5 * Hh.randn(g, B, T, C) for _ in range(3))
    w_raw, u, gy = Hh.randn(g, B, T, C) - 3.0, Hh.rand(g, H, N, lo=-1, hi=1), Hh.randn(g, B, T, C)
    rd, kd, vd, ud, gd = (x.to(dtype).to(DEV).contiguous() for x in (r, k, v, u, gy))
    ew = -torch.exp(w_raw.to(dtype).float()).to(DEV).contiguous()
    return rd, kd, vd, ew, ud, gd


def _outputs(dtype, B, T, C):
    big = lambda: torch.full((B, T, C), float("nan"), dtype=dtype, device=DEV)
    return big(), big(), big(), big(), torch.full((B, C), float("nan"), dtype=dtype, device=DEV)


@pytest.mark.parametrize("T", [100, 96])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_regular_entry_point_twice(dtype, T):
    import rwkv_cuda_b200 as R
    B, H, N = 2, 3, 64
    # bf16 with T a multiple of 16 sends the regular entry point to the chunked tensor-core kernels;
    # everything else runs the same general-shape kernel as the allocation-free entry point
    same_kernel = not (dtype == torch.bfloat16 and T % 16 == 0)
    C = H * N
    for call_no, seed in enumerate((11, 12)):     # two calls in a row, different data
        rd, kd, vd, ew, ud, gd = _inputs(dtype, B, T, H, N, seed)
        want = _outputs(dtype, B, T, C)
        R.ops.wkv6_backward(B, T, C, H, rd, kd, vd, ew, ud, gd, *want)
        got = _outputs(dtype, B, T, C)
        R.ops.wkv6_backward_noalloc(B, T, C, H, rd, kd, vd, ew, ud, gd, *got)
        torch.cuda.synchronize()
        for a, b, name in zip(got, want, ("gr", "gk", "gv", "gw", "gu")):
            assert torch.isfinite(a.float()).all(), f"call {call_no}: {name} has unwritten or non-finite elements"
            Hh.assert_close(a, b.double().cpu(), Hh.tol_for(dtype), f"call {call_no}: {name}")
            if same_kernel:   # same kernel, same arithmetic: bit for bit
                assert torch.equal(a, b), f"call {call_no}: {name} differs from the regular entry point"


def test_noalloc_refuses_oversized_problem():
    import rwkv_cuda_b200 as R
    from rwkv_cuda_b200 import _lib
    limit = _lib.lib().rwkvb200_wkv6_backward_noalloc_max_elems()
    B, T, H, N = 1, 16, 1, 64
    C = H * N
    rd, kd, vd, ew, ud, gd = _inputs(torch.bfloat16, B, T, H, N, 1)
    outs = _outputs(torch.bfloat16, B, T, C)
    # lie about T so that B*T*C exceeds the limit: the size check must fire before anything is launched
    T_big = limit // C + 1
    with pytest.raises(R.RwkvB200Error, match="exceeds the built-in scratch"):
        _lib.call("rwkvb200_wkv6_backward_noalloc", 1, B, T_big, C, H, rd.data_ptr(), kd.data_ptr(), vd.data_ptr(),
                  ew.data_ptr(), ud.data_ptr(), gd.data_ptr(), *(o.data_ptr() for o in outs), None)
