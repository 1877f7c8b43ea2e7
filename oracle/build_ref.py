"""TEST INFRASTRUCTURE ONLY.  Compiles the reference project's own CUDA kernels for sm_100 from a reference
checkout into oracle/_ref/, each with the reference's own nvcc flags, as checkers and on-box speed
comparisons:

    librwkv7_ref.so        rwkv7_fast_fused/cuda/rwkv7_statepassing_clampw.cu  (bf16, N=64, chunk 16;
                           flags of rwkv7_fast_fused/rwkv7_cuda_benchmark_state_passing.py:73)
    librwkv5_ref.so        wkv5_bf16/cuda/wkv5_cuda_v1b.cu                     (N=64; flags of wkv5_bf16/run.py:41-42)
    librwkv6state_ref.so   wkv6_state/cuda/wkv6state_cuda_v1a.cu               (N=64, T=256 baked in; wkv6_state/run.py:77-78)

Only the built libraries are kept (oracle/_ref/ is git-ignored); no reference source is copied.

    python oracle/build_ref.py [/path/to/RWKV-CUDA]      # or RWKV_CUDA_REF=/path/to/RWKV-CUDA
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "librwkv7_ref.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["--use_fast_math", "-O3", "-Xptxas", "-O3", "--extra-device-vectorization", "-Xcompiler", "-fPIC", "-shared"]
# library name -> (source inside the checkout, wrapper here, -D flags, needs the ATen headers)
TARGETS = {
    "librwkv7_ref.so": ("rwkv7_fast_fused/cuda/rwkv7_statepassing_clampw.cu", "ref_wrap.cu", ["-D_N_=64", "-D_CHUNK_LEN_=16"], False),
    "librwkv5_ref.so": ("wkv5_bf16/cuda/wkv5_cuda_v1b.cu", "ref_wrap_wkv5.cu", ["-D_N_=64"], True),
    "librwkv6state_ref.so": ("wkv6_state/cuda/wkv6state_cuda_v1a.cu", "ref_wrap_wkv6state.cu", ["-D_N_=64", "-D_T_=256"], True),
}


def checkout(ref=None):
    """The reference checkout: the argument, $RWKV_CUDA_REF, or the places a checkout is usually put."""
    for cand in (ref, os.environ.get("RWKV_CUDA_REF"), os.path.join(HERE, "..", "baseline", "_ref"),
                 os.path.join(HERE, "..", "..", "reference")):   # ... or a sibling directory `reference` of this repository
        if cand and os.path.exists(os.path.join(cand, "rwkv7_fast_fused", "cuda", "rwkv7_statepassing_clampw.cu")):
            return cand
    return None


def _aten_includes():
    from torch.utils.cpp_extension import include_paths
    return [f"-I{p}" for p in include_paths()]


def build(ref=None):
    """Builds what is out of date; returns the RWKV-7 library path, or None when neither a checkout nor a
    previously built library is present."""
    ref = checkout(ref)
    if ref is None:
        return LIB if os.path.exists(LIB) else None
    os.makedirs(OUT, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    for name, (rel, wrap, defs, aten) in TARGETS.items():
        src, wrap, lib = os.path.join(ref, rel), os.path.join(HERE, wrap), os.path.join(OUT, name)
        if not os.path.exists(src):
            continue
        if os.path.exists(lib) and os.path.getmtime(lib) > max(os.path.getmtime(src), os.path.getmtime(wrap)):
            continue
        inc = _aten_includes() + ["-std=c++17"] if aten else []
        subprocess.run([nvcc, *ARCH, *defs, *COMMON, *inc, src, wrap, "-o", lib, "-lcudart"], check=True)
    return LIB if os.path.exists(LIB) else None


if __name__ == "__main__":
    print(build(*sys.argv[1:2]))
