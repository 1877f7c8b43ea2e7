"""rwkv_cuda_b200: B200 (sm_100a) kernels for the WKV recurrences and depthwise_conv1d of
BlinkDL/RWKV-CUDA, behind that project's operator interface.

    ops        tensor-level forward/backward with the reference bindings' argument order
    load       stand-in for torch.utils.cpp_extension.load as the reference harnesses call it
    functions  torch.autograd.Function classes named as in the reference harnesses
    dist       batch sharding and the parameter-gradient all-reduce for multi-GPU runs
    host_pipeline  RWKV-7 forward+backward on operands that live in pinned host memory (streamed in batch slices)
"""
from . import _lib, ops, functions, dist, host_pipeline  # noqa: F401
from .load import load, parse_defines  # noqa: F401
from ._lib import RwkvB200Error  # noqa: F401

__all__ = ["ops", "functions", "dist", "host_pipeline", "load", "parse_defines", "RwkvB200Error"]
