"""CPU tier: the `load(...)` stand-in accepts the reference harnesses' calls."""
import pytest
import torch

import rwkv_cuda_b200 as R


def test_parse_defines():
    d = R.parse_defines(["-res-usage", "-D_N_=64", "-D_CHUNK_LEN_=16", "--use_fast_math", "-O3", "-Xptxas -O3",
                         "-D_FP32_", "-DTmax=768", "-DBF=8", "-DBB=2"])
    assert d == {"_N_": 64, "_CHUNK_LEN_": 16, "_FP32_": True, "Tmax": 768, "BF": 8, "BB": 2}


@pytest.mark.parametrize("name", ["wkv", "timex", "wkv5", "wkv5a", "wkv6", "wkv6state"])
def test_pybind_style_modules(name):
    m = R.load(name=name, sources=["cuda/x_op.cpp", "cuda/x.cu"], verbose=True,
               extra_cuda_cflags=["--use_fast_math", "-D_N_=64", "-D_T_=4096"], extra_cflags=["/wd4624"])
    assert callable(m.forward) and callable(m.backward)
    assert m.defines["_N_"] == 64


def test_head_size_flag_is_checked():
    m = R.load(name="wkv5", sources=[], extra_cuda_cflags=["-D_N_=64"])
    with pytest.raises(RuntimeError, match="head size 64"):
        m.forward(1, 4, 128, 1, *([torch.zeros(1)] * 6))


def test_torch_library_registration():
    flags = ["-res-usage", "-D_N_=64", "-D_CHUNK_LEN_=16", "--use_fast_math", "-O3"]
    for name in ("rwkv7_clampw", "rwkv7_state_clampw", "rwkv7_statepassing_clampw"):
        assert R.load(name=name, sources=[f"cuda/{name}.cu", f"cuda/{name}.cpp"], is_python_module=False,
                      verbose=True, extra_cuda_cflags=flags) is None
        ns = getattr(torch.ops, name)
        assert ns.forward is not None and ns.backward is not None
    # loading again with other flags (the harness's fp32 mode) rebinds instead of failing
    R.load(name="rwkv7_clampw", sources=[], is_python_module=False, extra_cflags=["-D_FP32_"],
           extra_cuda_cflags=flags + ["-D_FP32_"])


def test_unknown_extension_name():
    with pytest.raises(ValueError, match="unknown extension"):
        R.load(name="flash_attention", sources=[])


def test_reference_class_names_exist():
    for cls in ("WKV", "TimeX", "WKV_5", "WKV_5A", "WKV_6", "WKV_6STATE", "RWKV7_CLAMPW_CUDA_OP",
                "RWKV7_STATE_CLAMPW_CUDA_OP", "RWKV7_STATE_PASSING_CLAMPW_CUDA_OP"):
        assert issubclass(getattr(R.functions, cls), torch.autograd.Function)
