// Building blocks shared by the chunked (tensor-core) kernels: TF32 rounding, single-instruction
// approximations, bf16 pair conversion, cp.async, the optional phase counters (used by the RWKV-7
// tcgen05 kernels and by the 16-token RWKV-6 / RWKV-5 kernels) and the mma.sync m16n8k8 TF32 products
// with their fragment loaders (used by the RWKV-6 / RWKV-5 kernels, head size 64, chunks of 16 tokens).
//
// All contractions take operands rounded to TF32 and accumulate in fp32; states, decays and every
// elementwise step stay fp32.
#pragma once
#include "common.cuh"

namespace rwkvb200 {
namespace v7c {

constexpr int N = 64;     // head size
constexpr int L = 16;     // chunk length
constexpr int NT = 128;   // threads per CTA: 4 warps, warp w owns state rows 16w..16w+15
constexpr int PT = 72;    // pitch (floats) of token-major [16][64] operand arrays
constexpr int PK = 68;    // pitch (floats) of token-major arrays that are read along the token index
constexpr int PU = 24;    // pitch (floats) of the 16x16 matrices
constexpr int RP = 72;    // pitch (bf16 elements) of the staged [16][64] input tiles in the backward kernels
constexpr int PS = 68;    // pitch (floats) of the [16][64] output staging rows
constexpr float kWScale = -0.6065306597126334f;  // -exp(-1/2)
constexpr float kWScale2 = kWScale * 1.4426950408889634f;   // the same in log2 units: cumulative log-decays are kept base 2

// Round to TF32 (nearest, ties away from zero: what cvt.rna.tf32.f32 does) with two integer
// instructions.  The cvt form issues on the quarter-rate conversion pipe, which the four resident
// CTAs of an SM hit at the same time during operand preparation.
__device__ __forceinline__ uint32_t tf32(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }
// The same rounding for a value that only ever feeds a tensor-core operand: the tensor core reads the
// upper 19 bits of a TF32 operand register or shared-memory word and ignores the rest, so adding
// half a unit of the last kept place is enough (one instruction; results are bit-identical to tf32()).
__device__ __forceinline__ uint32_t tf32r(float x) { return __float_as_uint(x) + 0x1000u; }
__device__ __forceinline__ float tf32rf(float x) { return __uint_as_float(tf32r(x)); }

// Single-instruction approximations (flush-to-zero forms: no denormal fix-up code around them).
// Their arguments here are decays >= 6e-5, sums 1 + e^x and log-decays in [-10, 0].
__device__ __forceinline__ float fex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fexp(float x) { return fex2(x * 1.4426950408889634f); }
__device__ __forceinline__ float frcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// D += A(16x8, row) * B(8x8, col), TF32 in, fp32 accumulate.
// A: a0=(g,t) a1=(g+8,t) a2=(g,t+4) a3=(g+8,t+4); B: b0=(k=t,n=g) b1=(k=t+4,n=g);
// D: d0=(g,2t) d1=(g,2t+1) d2=(g+8,2t) d3=(g+8,2t+1)   with g = lane/4, t = lane%4.
__device__ __forceinline__ void mma8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                     uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Position of channel c (0..7) inside its group of 8 in a channel-permuted array: even channels
// first.  Reading positions (t, t+4) of such an array yields channels (2t, 2t+1), i.e. the
// permuted k order, with plain 32-bit loads.
__device__ __forceinline__ int perm8(int c) { return (c >> 1) + ((c & 1) << 2); }

// Key-channel relabelling used by the backward kernel.  The algorithm is equivariant under a
// permutation of the key index j applied to r, w, k, a, b, their gradients and the state columns,
// so inside each block of 16 key channels the kernel works on "logical" indices
//   logical = (real >> 1) + 8 * (real & 1)          real = 2 * (logical & 7) + (logical >> 3)
// which makes the two fragment rows a thread owns (g, g+8) the adjacent real channels (2g, 2g+1):
// every per-row access to the bf16 tiles, to W_t and to global memory is one 32- or 64-bit access.
__device__ __forceinline__ int key_logical(int real) { return (real & ~15) + ((real & 15) >> 1) + ((real & 1) << 3); }
__device__ __forceinline__ int key_real(int logical) { return (logical & ~15) + ((logical & 7) << 1) + ((logical >> 3) & 1); }
__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t x) {
    return make_float2(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
}
__device__ __forceinline__ uint32_t f2_to_bf16x2(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}

// Throughout, the contraction index inside one k-step of 8 is permuted so that MMA slot t maps
// to element 2t and slot t+4 to element 2t+1.  An accumulator tile (d0..d3) is then directly an
// A fragment (a0=d0, a1=d2, a2=d1, a3=d3), and B / A fragments read from shared memory are one
// 64-bit load of two adjacent elements.
__device__ __forceinline__ uint2 lds2(const float* p) { return *reinterpret_cast<const uint2*>(p); }

// acc[nt] (nt < NTILES) += Areg(16 x 8*KS) * B,  B read from a row-major [n][k] array `bm`
// (pitch `pb` floats): element (k, n) at bm[n*pb + k].  Areg holds KS k-steps of A fragments.
template <int NTILES, int KS>
__device__ __forceinline__ void gemm_rs(float (*acc)[4], const uint32_t (*areg)[4], const float* bm, int pb, int g,
                                        int t) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) {
            const uint2 b = lds2(bm + (nt * 8 + g) * pb + ks * 8 + 2 * t);
            mma8(acc[nt], areg[ks][0], areg[ks][1], areg[ks][2], areg[ks][3], b.x, b.y);
        }
}

// acc += (Ahi + Alo) * B with each B fragment loaded once (B as in gemm_rs).
template <int NTILES, int KS>
__device__ __forceinline__ void gemm_rs2(float (*acc)[4], const uint32_t (*ahi)[4], const uint32_t (*alo)[4],
                                         const float* bm, int pb, int g, int t) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) {
            const uint2 b = lds2(bm + (nt * 8 + g) * pb + ks * 8 + 2 * t);
            mma8(acc[nt], ahi[ks][0], ahi[ks][1], ahi[ks][2], ahi[ks][3], b.x, b.y);
            mma8(acc[nt], alo[ks][0], alo[ks][1], alo[ks][2], alo[ks][3], b.x, b.y);
        }
}

// B from a row-major [n][k] array whose k positions are channel-permuted (plain 32-bit reads).
template <int NTILES, int KS>
__device__ __forceinline__ void gemm_rs_plain(float (*acc)[4], const uint32_t (*areg)[4], const float* bm, int pb,
                                              int g, int t) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) {
            const float* p = bm + (nt * 8 + g) * pb + ks * 8 + t;
            mma8(acc[nt], areg[ks][0], areg[ks][1], areg[ks][2], areg[ks][3], __float_as_uint(p[0]), __float_as_uint(p[4]));
        }
}

// A fragments from a row-major [m][k] array whose k positions are channel-permuted.
template <int KS>
__device__ __forceinline__ void load_a_plain(uint32_t (*areg)[4], const float* am, int pa, int row0, int g, int t) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const float* lo = am + (row0 + g) * pa + ks * 8 + t;
        const float* hi = lo + 8 * pa;
        areg[ks][0] = __float_as_uint(lo[0]); areg[ks][1] = __float_as_uint(hi[0]);
        areg[ks][2] = __float_as_uint(lo[4]); areg[ks][3] = __float_as_uint(hi[4]);
    }
}

// A fragments of channel rows row0+g / row0+g+8 from a row-major [k][m] array whose m positions are
// channel-permuted (row0 a multiple of 8).
template <int KS>
__device__ __forceinline__ void load_a_kperm(uint32_t (*areg)[4], const float* am, int pa, int row0, int g, int t) {
    const int gp = perm8(g);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const float* p0 = am + (ks * 8 + 2 * t) * pa + row0 + gp;
        areg[ks][0] = __float_as_uint(p0[0]);
        areg[ks][1] = __float_as_uint(p0[8]);
        areg[ks][2] = __float_as_uint(p0[pa]);
        areg[ks][3] = __float_as_uint(p0[pa + 8]);
    }
}

// B from a row-major [k][n] array whose n positions are channel-permuted (element (k, n) at
// bm[k*pb + 8*(n/8) + perm8(n%8)]).
template <int NTILES, int KS>
__device__ __forceinline__ void gemm_rs_kperm(float (*acc)[4], const uint32_t (*areg)[4], const float* bm, int pb,
                                              int g, int t) {
    const int gp = perm8(g);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) {
            const uint32_t b0 = __float_as_uint(bm[(ks * 8 + 2 * t) * pb + nt * 8 + gp]);
            const uint32_t b1 = __float_as_uint(bm[(ks * 8 + 2 * t + 1) * pb + nt * 8 + gp]);
            mma8(acc[nt], areg[ks][0], areg[ks][1], areg[ks][2], areg[ks][3], b0, b1);
        }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int K>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(K) : "memory"); }

// Optional per-phase cycle counters (compile with -DRWKVB200_PHASE_CLOCKS; off in the shipped
// library): lane 0 of every warp of CTA (0,0) adds the cycles since its previous mark to
// g_phase_clocks[warp][phase].  Each translation unit that uses the marks has its own copy and
// exports a reader next to its kernel.
#ifdef RWKVB200_PHASE_CLOCKS
static __device__ unsigned long long g_phase_clocks[8][16];
#define WKV7_PHASE_BEGIN() long long phase_last_ = clock64()
#define WKV7_PHASE(k)                                                                              \
    do {                                                                                           \
        if (blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0) {                       \
            const long long now_ = clock64();                                                      \
            atomicAdd(&g_phase_clocks[threadIdx.x >> 5][k], (unsigned long long)(now_ - phase_last_)); \
            phase_last_ = now_;                                                                    \
        }                                                                                          \
    } while (0)
#define WKV7_PHASE_READER(name)                                                                    \
    extern "C" int name(unsigned long long* out64) {                                               \
        return (int)cudaMemcpyFromSymbol(out64, g_phase_clocks, sizeof(g_phase_clocks));           \
    }
#else
#define WKV7_PHASE_BEGIN()
#define WKV7_PHASE(k)
#define WKV7_PHASE_READER(name)
#endif

}  // namespace v7c
}  // namespace rwkvb200
