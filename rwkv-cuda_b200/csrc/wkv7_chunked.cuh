// Building blocks of the chunked (tensor-core) RWKV-7 kernels: head size 64, chunk of 16 tokens.
//
// Chunked form of the recurrence.  S is [value i][key j]; within a chunk of L = 16 tokens let
// W_t = prod_{tau<=t} d_tau (inclusive, per key channel), W_{-1} = 1, We = W_15, and
//   a~_t = a_t*W_{t-1}   r~_t = r_t*W_t   b~_s = b_s/W_s   k~_s = k_s/W_s   b^_s = b~_s*We   k^_s = k~_s*We
//   U_ab[s,t] = b~_s.a~_t (s<t)   U_ak[s,t] = k~_s.a~_t (s<t)   U_br[s,t] = b~_s.r~_t (s<=t)   U_kr[s,t] = k~_s.r~_t (s<=t)
//   T = (I - U_ab)^-1
// then with S0 the state at the start of the chunk, V = [v_t], SA = [sa_t], Y = [y_t] (64 x 16):
//   SA = (S0 A~ + V U_ak) T          Y = S0 R~ + SA U_br + V U_kr          S_end = S0 diag(We) + SA B^ + V K^
// The divisions by W are safe because the soft clamp keeps d >= 0.545, so W >= 0.545^16 = 6e-5.
//
// All contractions run on mma.sync m16n8k8 TF32 (operands rounded to TF32, fp32 accumulate);
// the state itself, the decays, the triangular inverse and every elementwise step stay fp32.
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

__device__ __forceinline__ uint32_t tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float tf32f(float x) { return __uint_as_float(tf32(x)); }

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

// A fragments (KS k-steps) of rows row0+g / row0+g+8 from a row-major [m][k] array (pitch pa).
template <int KS>
__device__ __forceinline__ void load_a(uint32_t (*areg)[4], const float* am, int pa, int row0, int g, int t) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const uint2 lo = lds2(am + (row0 + g) * pa + ks * 8 + 2 * t);
        const uint2 hi = lds2(am + (row0 + g + 8) * pa + ks * 8 + 2 * t);
        areg[ks][0] = lo.x; areg[ks][1] = hi.x; areg[ks][2] = lo.y; areg[ks][3] = hi.y;
    }
}

// Same product with B read from a row-major [k][n] array (pitch pb): element (k, n) at bm[k*pb + n].
template <int NTILES, int KS>
__device__ __forceinline__ void gemm_rs_kmaj(float (*acc)[4], const uint32_t (*areg)[4], const float* bm, int pb,
                                             int g, int t) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) {
            const uint32_t b0 = __float_as_uint(bm[(ks * 8 + 2 * t) * pb + nt * 8 + g]);
            const uint32_t b1 = __float_as_uint(bm[(ks * 8 + 2 * t + 1) * pb + nt * 8 + g]);
            mma8(acc[nt], areg[ks][0], areg[ks][1], areg[ks][2], areg[ks][3], b0, b1);
        }
}

// A fragments of rows row0+g / row0+g+8 from a row-major [k][m] array (pitch pa): element (m, k) at am[k*pa + m].
template <int KS>
__device__ __forceinline__ void load_a_kmaj(uint32_t (*areg)[4], const float* am, int pa, int row0, int g, int t) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const float* p0 = am + (ks * 8 + 2 * t) * pa + row0 + g;
        areg[ks][0] = __float_as_uint(p0[0]);
        areg[ks][1] = __float_as_uint(p0[8]);
        areg[ks][2] = __float_as_uint(p0[pa]);
        areg[ks][3] = __float_as_uint(p0[pa + 8]);
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

// accumulator tiles -> A fragments (rounded to TF32)
template <int KS>
__device__ __forceinline__ void acc_to_a(uint32_t (*areg)[4], const float (*acc)[4]) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        areg[ks][0] = tf32(acc[ks][0]); areg[ks][1] = tf32(acc[ks][2]);
        areg[ks][2] = tf32(acc[ks][1]); areg[ks][3] = tf32(acc[ks][3]);
    }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int K>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(K) : "memory"); }

// T = (I - U)^-1 for a strictly upper triangular 16x16 U (U[s][m], pitch PU), by back
// substitution in fp32; lane t (< 16) owns column t.  Result rounded to TF32 and stored
// transposed (Tt[t][s]) or, with NATURAL, as T[s][t].  Called by one full warp.
template <bool NATURAL = false>
__device__ __forceinline__ void tri_inverse(const float* U, float* Tt, int lane) {
    const int t = lane & 15;
    float col[L];
#pragma unroll
    for (int m = 0; m < L; ++m) col[m] = (m == t) ? 1.f : 0.f;
#pragma unroll
    for (int s = L - 2; s >= 0; --s) {
        // T[s,t] = sum_{m>s} U[s,m] T[m,t]   (zero for s >= t because col[m>t] = 0)
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int m = s + 1; m < L; ++m) {
            if ((m - s) & 1) acc0 = fmaf(U[s * PU + m], col[m], acc0);
            else acc1 = fmaf(U[s * PU + m], col[m], acc1);
        }
        if (s < t) col[s] = acc0 + acc1;
    }
    if (lane < 16) {
#pragma unroll
        for (int s = 0; s < L; ++s) Tt[NATURAL ? s * PU + t : t * PU + s] = tf32f(col[s]);
    }
}

}  // namespace v7c
}  // namespace rwkvb200
