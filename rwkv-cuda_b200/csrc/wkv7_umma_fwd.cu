// RWKV-7 forward, head size 64, bf16 activations: tcgen05 (5th-generation tensor core) kernel.
//
// Same chunked algorithm as wkv7_chunked_fwd.cu (symbols in wkv7_chunked.cuh), with the three
// K=64 / N>=32 products issued as tcgen05.mma (kind::tf32, M=64, cta_group::1): the tensor core
// reads its operands straight from shared memory (or, for the state, from tensor memory), so
// the B tiles no longer travel through the load/store pipe once per warp.
//
//   tensor memory (128 columns per CTA):  S [0,64)   fp32 state, rows = value i
//                                         X [64,96)  S [A~|R~]^T        (per chunk)
//                                         U [96,128) [B~;K~] [A~|R~]^T  (per chunk; rows 0-15 b~, 16-31 k~)
//   per chunk:   U, X  <- two MMA groups (K = 64) on the prepared operands            -> mbarrier 1
//                U to shared memory (masked), T = (I-U_ab)^-1, X to registers (the accumulator
//                fragment layout of tcgen05.ld 16x256b is that of mma.sync, so the small K=16
//                chain SA = (X_a + V U_ak) T, Y = X_r + SA U_br + V U_kr stays on mma.sync)
//                S  += [SA|V] [B~;K~]  (one MMA group, K = 32, accumulating in place)  -> mbarrier 2
//                S  <- S diag(We) through registers (tcgen05.ld / st), also the saved chunk state
// An M=64 accumulator occupies lanes 0-15 of each 32-lane quarter of tensor memory (row m at lane
// m%16 + 32*(m/16)), so warp w reads and writes rows 16w..16w+15, as in the mma.sync kernels.
//
// Shared-memory operands use the canonical K-major, unswizzled layout: 16-byte (4 x tf32) pieces
// of K; piece kc of row r at kc*LBO + r*16 bytes (8-row groups 128 bytes apart = SBO); LBO carries
// 16 bytes of padding so that the elementwise writers hit distinct banks.
// Inputs do not pass through shared memory: thread (channel pair p = lane, token group = warp) loads
// its 2 channels x 4 tokens of r, w, k, v, a, b as 32-bit bf16 pairs straight into registers, one
// chunk ahead (a warp reads the 128 contiguous bytes of one token), and writes the scaled operands
// from there.
// Every wait on an mbarrier is bounded; on expiry the kernel records an error code and leaves.
#include "wkv7_umma.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7u {

constexpr int kTmemCols = 128;
constexpr int kColS = 0, kColX = 64, kColU = 96;

__device__ int g_umma_error = 0;      // 0 = fine; otherwise which wait expired (1 or 2) in some CTA

struct Smem {
    static constexpr int kARt = 0;                                // [A~;R~]   16 pieces x LBO_T
    static constexpr int kBKt = kARt + 16 * LBO_T;                // [B~;K~]
    static constexpr int kBKc = kBKt + 16 * LBO_T + 1024;         // [b~|k~] by channel, 8 pieces x LBO_C (+ slack: BKt is read as 64 rows)
    static constexpr int kSAV = kBKc + 8 * LBO_C;                 // [SA|V] by channel
    static constexpr int kU = kSAV + 8 * LBO_C;                   // Uab Uak Ubr Ukr Tt, 5 x L*PU floats
    static constexpr int kWe = kU + 5 * L * PU * 4;               // [N] floats
    static constexpr int kHalf = kWe + N * 4;                     // [4][N] log-decay sums of the four token groups
    static constexpr int kBar = kHalf + 4 * N * 4;                // 2 mbarriers + tmem slot
    static constexpr int kBytes = kBar + 32;
};
static_assert(2 * L * PS * 4 <= 2 * 16 * LBO_T, "y/sa staging reuses the token-major operand arrays");

__global__ void __launch_bounds__(NT, 4)
wkv7u_forward_kernel(int T, int H, const float* __restrict__ s0_, const bf16* __restrict__ r_,
                     const bf16* __restrict__ w_, const bf16* __restrict__ k_, const bf16* __restrict__ v_,
                     const bf16* __restrict__ a_, const bf16* __restrict__ b_, bf16* __restrict__ y_,
                     float* __restrict__ sT_, float* __restrict__ ck_, float* __restrict__ sa_) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *ARt = smem + Smem::kARt, *BKt = smem + Smem::kBKt, *BKc = smem + Smem::kBKc, *SAV = smem + Smem::kSAV;
    float* Um = reinterpret_cast<float*>(smem + Smem::kU);
    float *Uab = Um, *Uak = Um + L * PU, *Ubr = Um + 2 * L * PU, *Ukr = Um + 3 * L * PU, *Tt = Um + 4 * L * PU;
    float* We = reinterpret_cast<float*>(smem + Smem::kWe);
    float* Hs = reinterpret_cast<float*>(smem + Smem::kHalf);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + Smem::kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 2);
    float* ystage = reinterpret_cast<float*>(ARt);
    float* sastage = reinterpret_cast<float*>(BKt);

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = warp * 16;
    const int C = H * N;
    const i64 tok0 = (i64)bb * T * C + hh * N;
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const int nchunks = T / L;
    float* ck = ck_ ? ck_ + (i64)(bb * H + hh) * nchunks * N * N : nullptr;
    const bf16* src[6] = {r_, w_, k_, v_, a_, b_};

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar + 1)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tw = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's quarter of tensor memory

    // initial state -> tensor memory (and saved as the start state of chunk 0)
    {
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

    const int lrow = tid >> 3, lseg = tid & 7;
    // raw inputs of the next chunk: nx[x][q] = channels (2*lane, 2*lane+1) of tensor x at token 4*warp + q
    uint32_t nx[6][4];
    auto fetch = [&](int c) {
        const i64 off = tok0 + (i64)(c * L + 4 * warp) * C + 2 * lane;
#pragma unroll
        for (int x = 0; x < 6; ++x)
#pragma unroll
            for (int q = 0; q < 4; ++q) nx[x][q] = __ldg(reinterpret_cast<const unsigned int*>(src[x] + off + (i64)q * C));
    };
    fetch(0);
    int fail = 0;

    WKV7_PHASE_BEGIN();
    for (int c = 0; c < nchunks; ++c) {
        const uint32_t par = c & 1;
        tc_fence_before();
        if (__syncthreads_or(fail)) break;
        tc_fence_after();
        WKV7_PHASE(0);   // top barrier
        // ---- prep: thread = (channel pair 2*lane, 2*lane+1; tokens 4*warp .. 4*warp+3) --------------
        {
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
            WKV7_PHASE(8);   // prep: log-decays of the token group
            *reinterpret_cast<float2*>(Hs + warp * N + j0) = make_float2(run0, run1);
            __syncthreads();
            WKV7_PHASE(9);   // prep: exchange barrier
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
        WKV7_PHASE(10);  // prep: scaled operands
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        if (c + 1 < nchunks) fetch(c + 1);   // the registers are free again: request the next chunk

        WKV7_PHASE(1);   // prep + barrier
        // ---- U = [B~;K~][A~|R~]^T and X = S [A~|R~]^T on the tensor core ------------------------
        if (tid == 0) {
            const uint32_t id32 = umma_idesc(32);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t bd = umma_desc(smem_u32(ARt) + ks * 2 * LBO_T, LBO_T);
                umma_ss(tmem + kColU, umma_desc(smem_u32(BKt) + ks * 2 * LBO_T, LBO_T), bd, id32, ks > 0);
                umma_ts(tmem + kColX, tmem + kColS + ks * 8, bd, id32, ks > 0);
            }
            umma_commit(bar);
        }
        if (!mbar_wait(bar, par)) fail = 1;
        tc_fence_after();

        WKV7_PHASE(2);   // U, X on the tensor core
        float X[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) tmem_ld8(X[nt], tw + kColX + nt * 8);
        if (warp < 2) {   // warp 0: rows b~ -> U_ab, U_br;  warp 1: rows k~ -> U_ak, U_kr
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
        tmem_wait_ld();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();

        WKV7_PHASE(3);   // U extraction, inverse, barrier
        // ---- the small chain on mma.sync, in registers --------------------------------------------
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
        __syncthreads();
        tc_fence_after();

        WKV7_PHASE(4);   // chain, staging, barrier
        // ---- S += [SA|V] [B~;K~] on the tensor core ---------------------------------------------
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
            __nv_bfloat162 p0 = __floats2bfloat162_rn(y0.x, y0.y), p1 = __floats2bfloat162_rn(y0.z, y0.w);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(y1.x, y1.y), p3 = __floats2bfloat162_rn(y1.z, y1.w);
            uint4 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
            pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
            *reinterpret_cast<uint4*>(y_ + off) = pk;
            if (sa_ != nullptr) {
                float4* d = reinterpret_cast<float4*>(sa_ + off);
                d[0] = *reinterpret_cast<const float4*>(sastage + lrow * PS + lseg * 8);
                d[1] = *reinterpret_cast<const float4*>(sastage + lrow * PS + lseg * 8 + 4);
            }
        }
        WKV7_PHASE(5);   // y, sa stores
        if (!mbar_wait(bar + 1, par)) fail = 2;
        tc_fence_after();

        WKV7_PHASE(6);   // wait for the state update
        // ---- S <- S diag(We); this is the start state of the next chunk ---------------------------
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
        WKV7_PHASE(7);   // decay scaling + checkpoint
    }

    if (fail && tid == 0) atomicMax(&g_umma_error, fail);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kTmemCols) : "memory");
}

WKV7_PHASE_READER(rwkvb200_phase_clocks_umma_fwd)

}  // namespace v7u

int wkv7_umma_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k,
                      const void* v, const void* a, const void* b, void* y, float* sT, float* s, float* sa,
                      cudaStream_t st) {
    using namespace v7u;
    cudaError_t e = cudaFuncSetAttribute(wkv7u_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_forward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7u_forward_kernel<<<grid, NT, Smem::kBytes, st>>>(T, H, s0, (const bf16*)r, (const bf16*)w, (const bf16*)k,
                                                         (const bf16*)v, (const bf16*)a, (const bf16*)b, (bf16*)y, sT, s,
                                                         sa);
    return check_launch("wkv7_forward(tcgen05)");
}

int wkv7_umma_error() {
    int h = 0;
    cudaMemcpyFromSymbol(&h, v7u::g_umma_error, sizeof(int));
    return h;
}

}  // namespace rwkvb200
