"""TEST INFRASTRUCTURE ONLY.  Compiles the reference project's own RWKV-7 state-passing kernel
(bf16, head size 64, chunk 16 -- the benchmark configuration) for sm_100 from the reference
checkout into oracle/_ref/librwkv7_ref.so, with the reference's own nvcc flags
(rwkv7_fast_fused/rwkv7_cuda_benchmark_state_passing.py:73).  Only the built library is kept
(oracle/_ref/ is git-ignored); no reference source is copied.

    python oracle/build_ref.py [/path/to/RWKV-CUDA]
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "librwkv7_ref.so")


def build(ref="/root/reference"):
    """Returns the library path, or None when no reference checkout is present."""
    src = os.path.join(ref, "rwkv7_fast_fused", "cuda", "rwkv7_statepassing_clampw.cu")
    if not os.path.exists(src):
        return LIB if os.path.exists(LIB) else None
    os.makedirs(OUT, exist_ok=True)
    wrap = os.path.join(HERE, "ref_wrap.cu")
    if os.path.exists(LIB) and os.path.getmtime(LIB) > max(os.path.getmtime(src), os.path.getmtime(wrap)):
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-D_N_=64", "-D_CHUNK_LEN_=16", "--use_fast_math", "-O3",
             "-Xptxas", "-O3", "--extra-device-vectorization", "-Xcompiler", "-fPIC", "-shared"]
    subprocess.run([nvcc, *flags, src, wrap, "-o", LIB, "-lcudart"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(*sys.argv[1:2]))
