// Shared device/host helpers for the rwkvb200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/rwkvb200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "rwkvb200 kernels are written for sm_100a (Blackwell B200) only"
#endif

namespace rwkvb200 {

using bf16 = __nv_bfloat16;
using i64 = long long;

// ---- element conversion -------------------------------------------------------------
__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
template <typename E> __device__ __forceinline__ E from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }

// hint: bring the line that holds *p into L1 (ties up no register, unlike a load issued early)
__device__ __forceinline__ void prefetch_l1(const void* p) {
    asm volatile("prefetch.global.L1 [%0];" ::"l"(__cvta_generic_to_global(p)));
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

// ---- error plumbing (host) ----------------------------------------------------------
void set_error(const char* fmt, ...);

#define RWKV_REQUIRE(cond, code, ...)          \
    do {                                       \
        if (!(cond)) {                         \
            rwkvb200::set_error(__VA_ARGS__);  \
            return (code);                     \
        }                                      \
    } while (0)

#define RWKV_NOTNULL(p) RWKV_REQUIRE((p) != nullptr, RWKVB200_ENULL, "argument '%s' is NULL", #p)

#define RWKV_ALIGNED(p, n) \
    RWKV_REQUIRE((reinterpret_cast<uintptr_t>(p) % (n)) == 0, RWKVB200_EALIGN, "argument '%s' is not %d-byte aligned", #p, (int)(n))

// Called after every launch: turns a launch-time CUDA error into a status code.
int check_launch(const char* what);

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// test hook (rwkvb200_test_disable_tensor_maps): true makes every tensor-map maker report failure, so that the
// paths that load without TMA run on a machine that has it
bool tensor_maps_disabled();

// smallest instantiated head-size capacity holding N (32, 64 or 128), or 0
inline int head_capacity(int N) { return N <= 0 ? 0 : N <= 32 ? 32 : N <= 64 ? 64 : N <= 128 ? 128 : 0; }

}  // namespace rwkvb200
