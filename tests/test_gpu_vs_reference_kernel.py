"""bf16 RWKV-7: the library's error against the fp64 oracle must be no worse than the error
of the reference project's own CUDA kernel on the same inputs (both within 2e-2)."""
import pytest
import torch

from oracle import wkv_oracle as O
from tests import helpers as Hh
from tests import ref_kernel

pytestmark = pytest.mark.gpu

# bf16 outputs carry a rounding floor of ~1.7e-3 for either kernel, so "no worse" is judged with
# a 10 % margin for the noise of that floor; fp32 state outputs are held to the bf16 tolerance
# and their errors are printed.
SLACK = 1.10


@pytest.mark.skipif(not ref_kernel.available(), reason="reference kernel library was not built (no reference checkout)")
@pytest.mark.parametrize("B,T,H", [(2, 1024, 4), (1, 256, 2)])
def test_error_no_worse_than_reference_kernel(B, T, H):
    import rwkv_cuda_b200 as R
    N = 64
    inp = Hh.v7_inputs(B, T, H, N, seed=42)
    bf = torch.bfloat16
    inp64 = {n: (x.to(bf).double() if n not in ("s0", "dsT") else x.double()) for n, x in inp.items()}
    want = Hh.v7_oracle(inp64, H)
    ours = ref_kernel.run(inp, H, R.ops.wkv7_forward, R.ops.wkv7_backward)
    ref = ref_kernel.run(inp, H, ref_kernel.forward, ref_kernel.backward)
    report = []
    for n in ("y", "dr", "dw", "dk", "dv", "da", "db", "sT", "ds0"):
        w64 = want[n]
        eo = O.err_ratio(w64, ours[n].double().cpu().reshape(w64.shape))
        er = O.err_ratio(w64, ref[n].double().cpu().reshape(w64.shape))
        report.append(f"{n}: ours {eo:.3e} reference kernel {er:.3e}")
        assert eo <= Hh.TOL_BF16, f"{n}: {eo:.3e} > 2e-2"
        if n not in ("sT", "ds0"):
            assert eo <= er * SLACK + 1e-6, f"{n}: ours {eo:.3e} worse than the reference kernel {er:.3e}"
    print("\n".join(report))
