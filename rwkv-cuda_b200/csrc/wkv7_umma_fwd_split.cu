// RWKV-7 forward, head size 64, bf16 activations: the tcgen05 kernel of wkv7_umma_fwd.cu as a
// producer/consumer pair, for launches that put at most two (batch, head) units on an SM
// (strong scaling over GPUs at a small batch per GPU).  110 registers, 86 KB: two CTAs fit an SM.
//
// With one CTA per SM the time of the forward is the length of one unit's chain of chunks, and half
// of every chunk in wkv7_umma_fwd.cu does not depend on the state: operand preparation, the U
// matrices (their tcgen05.mma group and its read-out) and the 16x16 inverse.  Here four producer
// warps do that work one chunk ahead into a second operand set, while the four consumer warps, who
// own the state in tensor memory, run X = S [A~|R~]^T, the small chain, the state update and the
// decay scaling.  One CTA-wide barrier per chunk hands the finished set over and returns the other;
// inside a group the barriers are named barriers of 128 threads.  Tensor memory as in
// wkv7_umma_fwd.cu (S [0,64), X [64,96), U [96,128)): U is written and read by the producers only,
// X and S by the consumers only; each group issues its own tcgen05.mma and waits on its own mbarrier.
// Same arithmetic and order as wkv7_umma_fwd.cu: identical results.
// Every mbarrier wait is bounded; a wait that expires is recorded, the loop ends at the next
// hand-over barrier (taken by all 256 threads), tensor memory is freed and the kernel returns.
#include "wkv7_umma.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7us {

using namespace v7u;

constexpr int kTmemCols = 128;
constexpr int kColS = 0, kColX = 64, kColU = 96;
constexpr int NTS = 2 * NT;   // 8 warps: consumers 0-3, producers 4-7

__device__ int g_umma_split_error = 0;   // 0 = fine; otherwise 20 + which wait expired

struct SetMap {                                                  // one operand set, byte offsets
    static constexpr int kARt = 0;                                // [A~;R~]   16 pieces x LBO_T (reused as y staging)
    static constexpr int kBKt = kARt + 16 * LBO_T;                // [B~;K~]                       (reused as sa staging)
    static constexpr int kBKc = kBKt + 16 * LBO_T + 1024;         // [b~|k~] by channel, 8 pieces x LBO_C (+ slack: BKt is read as 64 rows)
    static constexpr int kSAV = kBKc + 8 * LBO_C;                 // [SA|V] by channel
    static constexpr int kU = kSAV + 8 * LBO_C;                   // Uab Uak Ubr Ukr Tt, 5 x L*PU floats
    static constexpr int kWe = kU + 5 * L * PU * 4;               // [N] floats
    static constexpr int kBytes = kWe + N * 4;
};
struct Smem {
    static constexpr int kSets = 0;
    static constexpr int kHs = 2 * SetMap::kBytes;                // [4][N] log-decay sums of the token groups
    static constexpr int kBar = kHs + 4 * N * 4;                  // 3 mbarriers (U, X, state update) + tmem slot
    static constexpr int kBytes = kBar + 32;
};
static_assert(SetMap::kBytes % 128 == 0, "operand sets keep the 128-byte alignment of their first array");
static_assert(2 * L * PS * 4 <= 2 * 16 * LBO_T, "y/sa staging reuses the token-major operand arrays");

__global__ void __launch_bounds__(NTS, 2)
wkv7us_forward_kernel(int T, int H, const float* __restrict__ s0_, const bf16* __restrict__ r_,
                      const bf16* __restrict__ w_, const bf16* __restrict__ k_, const bf16* __restrict__ v_,
                      const bf16* __restrict__ a_, const bf16* __restrict__ b_, bf16* __restrict__ y_,
                      float* __restrict__ sT_, float* __restrict__ ck_, float* __restrict__ sa_) {
    extern __shared__ __align__(128) unsigned char smem[];
    float* Hs = reinterpret_cast<float*>(smem + Smem::kHs);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + Smem::kBar);   // [0] U (producers)  [1] state update  [2] X (consumers)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 3);

    const int hh = blockIdx.x, bb = blockIdx.y;
    const bool producer = threadIdx.x >= NT;
    // group-local indices: each group of four warps is laid out like the CTA of wkv7_umma_fwd.cu
    const int tid = threadIdx.x & (NT - 1), warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = warp * 16;
    const int C = H * N;
    const i64 tok0 = (i64)bb * T * C + hh * N;
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const int nchunks = T / L;
    float* ck = ck_ ? ck_ + (i64)(bb * H + hh) * nchunks * N * N : nullptr;
    const bf16* src[6] = {r_, w_, k_, v_, a_, b_};
    auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(producer ? 2 : 1) : "memory"); };

    if (threadIdx.x == 0) {
#pragma unroll
        for (int q = 0; q < 3; ++q) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar + q)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tw = tmem + ((uint32_t)(warp * 32) << 16);   // warps w and w+4 share tensor-memory quarter w

    int fail = 0;
    // raw inputs of the next chunk to prepare (producers): nx[x][q] = channels (2*lane, 2*lane+1) of
    // tensor x at token 4*warp + q
    uint32_t nx[6][4];
    auto fetch = [&](int c) {
        const i64 off = tok0 + (i64)(c * L + 4 * warp) * C + 2 * lane;
#pragma unroll
        for (int x = 0; x < 6; ++x)
#pragma unroll
            for (int q = 0; q < 4; ++q) nx[x][q] = __ldg(reinterpret_cast<const unsigned int*>(src[x] + off + (i64)q * C));
    };

    // ---- producers: operands, U and T = (I - U_ab)^-1 of chunk c into its set --------------------
    auto produce = [&](int c) {
        unsigned char* set = smem + Smem::kSets + (c & 1) * SetMap::kBytes;
        unsigned char *ARt = set + SetMap::kARt, *BKt = set + SetMap::kBKt, *BKc = set + SetMap::kBKc, *SAV = set + SetMap::kSAV;
        float* Um = reinterpret_cast<float*>(set + SetMap::kU);
        float *Uab = Um, *Uak = Um + L * PU, *Ubr = Um + 2 * L * PU, *Ukr = Um + 3 * L * PU, *Tt = Um + 4 * L * PU;
        float* We = reinterpret_cast<float*>(set + SetMap::kWe);
        {   // thread = (channel pair 2*lane, 2*lane+1; tokens 4*warp .. 4*warp+3)
            const int j0 = 2 * lane, t0 = 4 * warp;
            float cs[4][2];
            float run0 = 0.f, run1 = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 x = bf16x2_to_f2(nx[1][q]);
                run0 = fmaf(kWScale2, frcp(1.f + fexp(-x.x)), run0);
                run1 = fmaf(kWScale2, frcp(1.f + fexp(-x.y)), run1);
                cs[q][0] = run0; cs[q][1] = run1;
            }
            *reinterpret_cast<float2*>(Hs + warp * N + j0) = make_float2(run0, run1);
            group_sync();
            float base0 = 0.f, base1 = 0.f, tot0 = 0.f, tot1 = 0.f;
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
                const float2 h = *reinterpret_cast<const float2*>(Hs + gq * N + j0);
                if (gq < warp) { base0 += h.x; base1 += h.y; }
                tot0 += h.x; tot1 += h.y;
            }
            if (warp == 0) *reinterpret_cast<float2*>(We + j0) = make_float2(fex2(tot0), fex2(tot1));
            float wp0 = fex2(base0), wp1 = fex2(base1);
            float bt[4][2], kt[4][2], vv[4][2];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int tt = t0 + q;
                const float lam0 = base0 + cs[q][0], lam1 = base1 + cs[q][1];
                const float wt0 = fex2(lam0), wt1 = fex2(lam1), iw0 = fex2(-lam0), iw1 = fex2(-lam1);
                const float2 r2 = bf16x2_to_f2(nx[0][q]), k2 = bf16x2_to_f2(nx[2][q]), v2 = bf16x2_to_f2(nx[3][q]);
                const float2 a2 = bf16x2_to_f2(nx[4][q]), b2 = bf16x2_to_f2(nx[5][q]);
                bt[q][0] = tf32rf(b2.x * iw0); bt[q][1] = tf32rf(b2.y * iw1);
                kt[q][0] = tf32rf(k2.x * iw0); kt[q][1] = tf32rf(k2.y * iw1);
                vv[q][0] = v2.x; vv[q][1] = v2.y;
                *reinterpret_cast<float2*>(ARt + canon(tt, j0, LBO_T)) = make_float2(tf32rf(a2.x * wp0), tf32rf(a2.y * wp1));
                *reinterpret_cast<float2*>(ARt + canon(16 + tt, j0, LBO_T)) = make_float2(tf32rf(r2.x * wt0), tf32rf(r2.y * wt1));
                *reinterpret_cast<float2*>(BKt + canon(tt, j0, LBO_T)) = make_float2(bt[q][0], bt[q][1]);
                *reinterpret_cast<float2*>(BKt + canon(16 + tt, j0, LBO_T)) = make_float2(kt[q][0], kt[q][1]);
                wp0 = wt0; wp1 = wt1;
            }
            // by channel: row j, K index = token (b~: 0..15, k~: 16..31; v: 16..31 of SAV)
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                *reinterpret_cast<float4*>(BKc + canon(j0 + ch, t0, LBO_C)) = make_float4(bt[0][ch], bt[1][ch], bt[2][ch], bt[3][ch]);
                *reinterpret_cast<float4*>(BKc + canon(j0 + ch, 16 + t0, LBO_C)) = make_float4(kt[0][ch], kt[1][ch], kt[2][ch], kt[3][ch]);
                *reinterpret_cast<float4*>(SAV + canon(j0 + ch, 16 + t0, LBO_C)) = make_float4(vv[0][ch], vv[1][ch], vv[2][ch], vv[3][ch]);
            }
        }
        proxy_fence();
        tc_fence_before();
        group_sync();
        tc_fence_after();
        if (c + 1 < nchunks) fetch(c + 1);   // the registers are free again: request the next chunk

        // U = [B~;K~][A~|R~]^T on the tensor core
        if (tid == 0) {
            const uint32_t id32 = umma_idesc(32);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                umma_ss(tmem + kColU, umma_desc(smem_u32(BKt) + ks * 2 * LBO_T, LBO_T),
                        umma_desc(smem_u32(ARt) + ks * 2 * LBO_T, LBO_T), id32, ks > 0);
            umma_commit(bar);
        }
        if (warp < 2) {   // warp 0: rows b~ -> U_ab, U_br;  warp 1: rows k~ -> U_ak, U_kr
            if (!fail && !mbar_wait(bar, c & 1)) fail = 1;
            tc_fence_after();
            float U[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) tmem_ld8(U[nt], tw + kColU + nt * 8);
            tmem_wait_ld();
            float* dstA = warp == 0 ? Uab : Uak;     // vs a~: strictly upper
            float* dstR = warp == 0 ? Ubr : Ukr;     // vs r~: upper incl. diagonal
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int s = g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                    const float ua = s < tt ? U[nt][e] : 0.f, ur = s <= tt ? U[2 + nt][e] : 0.f;
                    if (warp == 0) dstA[s * PU + tt] = ua; else dstA[tt * PU + s] = tf32rf(ua);
                    dstR[tt * PU + s] = tf32rf(ur);
                }
            if (warp == 0) {
                __syncwarp();
                tri_inverse(Uab, Tt, lane);
            }
        }
    };

    // ---- consumers: chunk c from its operand set --------------------------------------------------
    auto consume = [&](int c) {
        const uint32_t par = c & 1;
        unsigned char* set = smem + Smem::kSets + (c & 1) * SetMap::kBytes;
        unsigned char *ARt = set + SetMap::kARt, *BKt = set + SetMap::kBKt, *BKc = set + SetMap::kBKc, *SAV = set + SetMap::kSAV;
        float* Um = reinterpret_cast<float*>(set + SetMap::kU);
        float *Uak = Um + L * PU, *Ubr = Um + 2 * L * PU, *Ukr = Um + 3 * L * PU, *Tt = Um + 4 * L * PU;
        const float* We = reinterpret_cast<const float*>(set + SetMap::kWe);
        float* ystage = reinterpret_cast<float*>(ARt);
        float* sastage = reinterpret_cast<float*>(BKt);
        const int lrow = tid >> 3, lseg = tid & 7;

        // X = S [A~|R~]^T on the tensor core
        if (tid == 0) {
            const uint32_t id32 = umma_idesc(32);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                umma_ts(tmem + kColX, tmem + kColS + ks * 8, umma_desc(smem_u32(ARt) + ks * 2 * LBO_T, LBO_T), id32, ks > 0);
            umma_commit(bar + 2);
        }
        if (!fail && !mbar_wait(bar + 2, par)) fail = 3;
        tc_fence_after();
        float X[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) tmem_ld8(X[nt], tw + kColX + nt * 8);
        tmem_wait_ld();

        // the small chain on mma.sync, in registers
        uint32_t vreg[2][4], xreg[2][4], sareg[2][4];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {   // A[m=i][k=s] = v_s[i] from the by-channel operand (K index 16+s)
            const int s = 16 + ks * 8 + 2 * t;
            vreg[ks][0] = *reinterpret_cast<const uint32_t*>(SAV + canon(row0 + g, s, LBO_C));
            vreg[ks][1] = *reinterpret_cast<const uint32_t*>(SAV + canon(row0 + g + 8, s, LBO_C));
            vreg[ks][2] = *reinterpret_cast<const uint32_t*>(SAV + canon(row0 + g, s + 1, LBO_C));
            vreg[ks][3] = *reinterpret_cast<const uint32_t*>(SAV + canon(row0 + g + 8, s + 1, LBO_C));
        }
        gemm_rs<2, 2>(X, vreg, Uak, PU, g, t);           // X_a += V U_ak
        acc_to_a<2>(xreg, X);
        float SA[2][4] = {};
        gemm_rs<2, 2>(SA, xreg, Tt, PU, g, t);           // SA = X_a T
        acc_to_a<2>(sareg, SA);
        gemm_rs<2, 2>(X + 2, sareg, Ubr, PU, g, t);      // Y = X_r + SA U_br + V U_kr
        gemm_rs<2, 2>(X + 2, vreg, Ukr, PU, g, t);

        // SA -> by-channel operand (K index = token), y / sa -> staging
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int s = nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(SAV + canon(row0 + g, s, LBO_C)) = make_float2(tf32rf(SA[nt][0]), tf32rf(SA[nt][1]));
            *reinterpret_cast<float2*>(SAV + canon(row0 + g + 8, s, LBO_C)) = make_float2(tf32rf(SA[nt][2]), tf32rf(SA[nt][3]));
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                ystage[tt * PS + i] = X[2 + nt][e];
                sastage[tt * PS + i] = SA[nt][e];
            }
        }
        proxy_fence();
        tc_fence_before();
        group_sync();
        tc_fence_after();

        // S += [SA|V] [B~;K~] on the tensor core
        if (tid == 0) {
            const uint32_t id64 = umma_idesc(64);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                umma_ss(tmem + kColS, umma_desc(smem_u32(SAV) + ks * 2 * LBO_C, LBO_C),
                        umma_desc(smem_u32(BKc) + ks * 2 * LBO_C, LBO_C), id64, 1);
            umma_commit(bar + 1);
        }
        {   // meanwhile: full-row stores of y and sa
            const i64 off = tok0 + (i64)(c * L + lrow) * C + lseg * 8;
            const float4 y0 = *reinterpret_cast<const float4*>(ystage + lrow * PS + lseg * 8);
            const float4 y1 = *reinterpret_cast<const float4*>(ystage + lrow * PS + lseg * 8 + 4);
            uint4 pk;
            pk.x = f2_to_bf16x2(y0.x, y0.y); pk.y = f2_to_bf16x2(y0.z, y0.w);
            pk.z = f2_to_bf16x2(y1.x, y1.y); pk.w = f2_to_bf16x2(y1.z, y1.w);
            *reinterpret_cast<uint4*>(y_ + off) = pk;
            if (sa_ != nullptr) {
                float4* d = reinterpret_cast<float4*>(sa_ + off);
                d[0] = *reinterpret_cast<const float4*>(sastage + lrow * PS + lseg * 8);
                d[1] = *reinterpret_cast<const float4*>(sastage + lrow * PS + lseg * 8 + 4);
            }
        }
        if (!fail && !mbar_wait(bar + 1, par)) fail = 2;
        tc_fence_after();

        // S <- S diag(We); this is the start state of the next chunk
        float* dst = (c + 1 < nchunks) ? (ck ? ck + (i64)(c + 1) * N * N : nullptr) : (sT_ ? sT_ + sbase : nullptr);
        float Sd[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) tmem_ld8(Sd[nt], tw + kColS + nt * 8);
        tmem_wait_ld();
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float2 we = *reinterpret_cast<const float2*>(We + nt * 8 + 2 * t);
            Sd[nt][0] *= we.x; Sd[nt][1] *= we.y; Sd[nt][2] *= we.x; Sd[nt][3] *= we.y;
            tmem_st8(tw + kColS + nt * 8, Sd[nt]);
            if (dst != nullptr) {
                *reinterpret_cast<float2*>(dst + (row0 + g) * N + nt * 8 + 2 * t) = make_float2(Sd[nt][0], Sd[nt][1]);
                *reinterpret_cast<float2*>(dst + (row0 + g + 8) * N + nt * 8 + 2 * t) = make_float2(Sd[nt][2], Sd[nt][3]);
            }
        }
        tmem_wait_st();
    };

    if (producer) {
        fetch(0);
        produce(0);
    } else {
        // initial state -> tensor memory (and saved as the start state of chunk 0)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float2 lo = make_float2(0.f, 0.f), hi = lo;
            if (s0_ != nullptr) {
                lo = *reinterpret_cast<const float2*>(s0_ + sbase + (row0 + g) * N + nt * 8 + 2 * t);
                hi = *reinterpret_cast<const float2*>(s0_ + sbase + (row0 + g + 8) * N + nt * 8 + 2 * t);
            }
            const float d[4] = {lo.x, lo.y, hi.x, hi.y};
            tmem_st8(tw + kColS + nt * 8, d);
            if (ck != nullptr) {
                *reinterpret_cast<float2*>(ck + (row0 + g) * N + nt * 8 + 2 * t) = lo;
                *reinterpret_cast<float2*>(ck + (row0 + g + 8) * N + nt * 8 + 2 * t) = hi;
            }
        }
        tmem_wait_st();
    }

    for (int c = 0; c < nchunks; ++c) {
        // hand-over: the set of chunk c is complete (producers), the other set and the state are
        // final (consumers); also the point where a recorded failure ends the loop for everybody
        tc_fence_before();
        const int any_fail = __syncthreads_or(fail);
        tc_fence_after();
        if (any_fail) break;
        if (producer) {
            if (c + 1 < nchunks) produce(c + 1);
        } else {
            consume(c);
        }
    }

    if (fail) atomicMax(&g_umma_split_error, 20 + fail);
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kTmemCols) : "memory");
}

}  // namespace v7us

int wkv7_umma_split_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k,
                            const void* v, const void* a, const void* b, void* y, float* sT, float* s, float* sa,
                            cudaStream_t st) {
    using namespace v7us;
    cudaError_t e = cudaFuncSetAttribute(wkv7us_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_forward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7us_forward_kernel<<<grid, NTS, Smem::kBytes, st>>>(T, H, s0, (const bf16*)r, (const bf16*)w, (const bf16*)k,
                                                           (const bf16*)v, (const bf16*)a, (const bf16*)b, (bf16*)y, sT,
                                                           s, sa);
    return check_launch("wkv7_forward(tcgen05, producer/consumer)");
}

int wkv7_umma_split_error() {
    int h = 0;
    cudaMemcpyFromSymbol(&h, v7us::g_umma_split_error, sizeof(int));
    return h;
}

}  // namespace rwkvb200
