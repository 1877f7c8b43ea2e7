// RWKV-7 forward, head size 64, bf16 activations: chunks of 32 tokens, every product on tcgen05.
//
// One CTA of 4 warps per (batch, head), persistent over the sequence, three CTAs per SM.  Per chunk
// (symbols and layouts in wkv7_l32.cuh):
//   1. operand preparation from registers (the chunk was fetched while the previous one ran)
//   2. U = [B~;K~][A~;R~]^T                                   tcgen05, -> mbarrier 0
//   3. U to shared memory (masked, TF32), inverses of the two 16x16 diagonal blocks of I - U_ab   CUDA cores
//   4. one warp issues the whole dependent chain, accumulators feeding the next product straight from
//      tensor memory:
//        X = S [A~;R~]^T      Z = X_a + V U_ak      SA = Z T (T applied as D0 + D0 N1 D0, blocks of 16 tokens)
//        Y = X_r + SA U_br + V U_kr                                                                  -> mbarrier 1
//      (between a product and a consumer of its accumulator the issuing warp waits on its own mbarrier)
//        S += SA B~ + V K~                                                                       -> mbarrier 2
//   5. Y -> bf16 -> global (while the state update runs), then S <- S diag(We) through registers,
//      which is also where the chunk-start state of the next chunk is saved.
// Tensor memory: 128 columns (S | U then X) + 32 columns (SA), as two allocations; three CTAs use 480
// of the SM's 512 columns, and shared memory (69 KB) keeps a fourth CTA away.
// Saved for the backward: the state at the start of every 32-token chunk, [chunk][i][j] per
// (batch, head), as s[b][h][c] of the caller's (B,H,T/16,64,64) buffer, c < ceil(T/32); `sa` is not used.
// T may be any multiple of 16: a last half chunk is padded with neutral tokens.
#include "wkv7_l32.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7x {

constexpr int FNT = 128;   // threads
constexpr int FTPW = 8;    // tokens per warp in operand preparation

__device__ int g_l32_fwd_error = 0;   // 0 = fine; otherwise which wait expired in some CTA

struct FwdSmem {
    static constexpr int kAR = 0;
    static constexpr int kBK = kAR + ARR64;
    static constexpr int kV = kBK + ARR64;              // [32][64] v_t
    static constexpr int kUak = kV + ARR32;             // [32][32] each
    static constexpr int kUbr = kUak + HALF32;
    static constexpr int kUkr = kUbr + HALF32;
    static constexpr int kD0 = kUkr + HALF32;           // diag(T00, T11)
    static constexpr int kN1 = kD0 + HALF32;            // upper right block of U_ab
    static constexpr int kUab = kN1 + HALF32;           // plain [32][UPITCH]
    static constexpr int kWe = kUab + 32 * UPITCH * 4;  // [64]
    static constexpr int kHs = kWe + 64 * 4;            // [4][64]
    static constexpr int kY = kHs + 4 * 64 * 4;         // bf16 [32][72]
    static constexpr int kBar = kY + 32 * 72 * 2;       // 4 mbarriers + 2 tmem slots
    static constexpr int kBytes = kBar + 64 + 1024;     // + slack to start on a 1024-byte boundary
};
static_assert(FwdSmem::kUab % 16 == 0 && FwdSmem::kWe % 16 == 0 && FwdSmem::kY % 16 == 0 && FwdSmem::kBar % 8 == 0, "alignment");
static_assert(FwdSmem::kBytes * 4 > 227 * 1024, "a fourth CTA per SM would exhaust tensor memory");

__global__ void __launch_bounds__(FNT, 3)
wkv7x_forward_kernel(int T, int H, const float* __restrict__ s0_, const bf16* __restrict__ r_,
                     const bf16* __restrict__ w_, const bf16* __restrict__ k_, const bf16* __restrict__ v_,
                     const bf16* __restrict__ a_, const bf16* __restrict__ b_, bf16* __restrict__ y_,
                     float* __restrict__ sT_, float* __restrict__ ck_, int test_expire) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // the swizzle acts on address bits
    unsigned char *AR = smem + FwdSmem::kAR, *BK = smem + FwdSmem::kBK, *Vs = smem + FwdSmem::kV;
    unsigned char *Uak = smem + FwdSmem::kUak, *Ubr = smem + FwdSmem::kUbr, *Ukr = smem + FwdSmem::kUkr;
    unsigned char *D0 = smem + FwdSmem::kD0, *N1 = smem + FwdSmem::kN1;
    float* Uab = reinterpret_cast<float*>(smem + FwdSmem::kUab);
    float* We = reinterpret_cast<float*>(smem + FwdSmem::kWe);
    float* Hs = reinterpret_cast<float*>(smem + FwdSmem::kHs);
    bf16* ystage = reinterpret_cast<bf16*>(smem + FwdSmem::kY);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + FwdSmem::kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 4);

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // warp-uniform for the compiler too
    const int row0 = warp * 16;
    const int C = H * 64;
    const i64 tok0 = (i64)bb * T * C + hh * 64;
    const i64 sbase = (i64)(bb * H + hh) * 64 * 64;
    const int nchunks = (T + LC - 1) / LC;
    float* ck = ck_ ? ck_ + (i64)(bb * H + hh) * (T / 16) * 64 * 64 : nullptr;   // block [b][h] of the caller's (B,H,T/16,N,N) buffer
    const bf16* src[6] = {r_, w_, k_, v_, a_, b_};

    if (tid == 0) {
        mbar_init(bar); mbar_init(bar + 1); mbar_init(bar + 2); mbar_init(bar + 3);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 32;" ::"r"(smem_u32(tmem_slot + 1)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmS = __shfl_sync(0xffffffffu, tmem_slot[0], 0), tmX = tmS + 64, tmSA = __shfl_sync(0xffffffffu, tmem_slot[1], 0);
    const uint32_t lead = elect_one();
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;   // this warp's quarter of tensor memory
    const uint32_t arA = smem_u32(AR), bkA = smem_u32(BK), vA = smem_u32(Vs);
    const uint32_t uakA = smem_u32(Uak), ubrA = smem_u32(Ubr), ukrA = smem_u32(Ukr);
    const uint32_t d0A = smem_u32(D0), n1A = smem_u32(N1);
    for (int i = tid; i < 2 * HALF32 / 4; i += FNT) reinterpret_cast<float*>(D0)[i] = 0.f;   // D0 and N1: the blocks never written stay zero

    // initial state -> tensor memory (and saved as the start state of chunk 0)
    {
        float Sd[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float2 lo = make_float2(0.f, 0.f), hi = lo;
            if (s0_ != nullptr) {
                lo = *reinterpret_cast<const float2*>(s0_ + sbase + (row0 + g) * 64 + nt * 8 + 2 * t);
                hi = *reinterpret_cast<const float2*>(s0_ + sbase + (row0 + g + 8) * 64 + nt * 8 + 2 * t);
            }
            Sd[nt][0] = lo.x; Sd[nt][1] = lo.y; Sd[nt][2] = hi.x; Sd[nt][3] = hi.y;
            if (ck != nullptr) {
                *reinterpret_cast<float2*>(ck + (row0 + g) * 64 + nt * 8 + 2 * t) = lo;
                *reinterpret_cast<float2*>(ck + (row0 + g + 8) * 64 + nt * 8 + 2 * t) = hi;
            }
        }
        tmem_st_tiles<8>(tmS + lane_off, Sd);
        tmem_wait_st();
    }

    RawChunk<6, FTPW> raw;
    fetch_chunk<6, FTPW>(raw, src, tok0, C, 0, T, warp, lane);
    int fail = 0;
    ChainSync cs{bar + 3, 0, 0};   // used by warp 0 only

    WKV7_PHASE_BEGIN();
    for (int c = 0; c < nchunks; ++c) {
        const uint32_t par = c & 1;
        const int valid = min(LC, T - c * LC);
        tc_fence_before();
        if (__syncthreads_or(fail)) break;
        tc_fence_after();
        WKV7_PHASE(0);   // top barrier
        // ---- 1. operands ---------------------------------------------------------------------------
        prepare_operands<6, FTPW, 4>(raw, valid, AR, BK, Vs, HALF32, nullptr, 0, We, Hs, nullptr, warp, lane);
        WKV7_PHASE(1);   // operand preparation
        proxy_fence();
        WKV7_PHASE(11);  // proxy fence
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        WKV7_PHASE(12);  // barrier
        WKV7_PHASE(2);   // barrier, fetch issue
        // ---- 2. U ------------------------------------------------------------------------------------
        if (warp == 0 && !(test_expire && c == 0)) {
            issue_u(tmX, arA, bkA, lead);
            mma_commit(bar, lead);
        }
        if (!mbar_wait(bar, par, test_expire ? (1 << 10) : (1 << 20))) fail = 1;
        tc_fence_after();
        WKV7_PHASE(3);   // U on the tensor core
        // ---- 3. masked U, inverse ----------------------------------------------------------------------
        {
            float u[8][4];
            tmem_ld_tiles<8>(u, tmX + lane_off);
            tmem_wait_ld();
            scatter_u(u, warp, lane, Uab, N1, Uak, Ubr, Ukr);
        }
        tc_fence_before();
        __syncthreads();
        WKV7_PHASE(4);   // masked U to shared memory
        if (warp < 2) tri_inverse16<UPITCH>(Uab + 16 * warp * (UPITCH + 1), D0, 16 * warp, lane);
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        WKV7_PHASE(5);   // inverse
        // ---- 4. the dependent chain --------------------------------------------------------------------
        if (warp == 0) {
            const uint32_t id64 = idesc64(64, 0, 0);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // X = S [A~;R~]^T
                mma_ts(tmX, tmS + ks * 8, desc_k(arA, 0, ks * 8, HALF64), id64, ks > 0, lead);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // Z = X_a + V U_ak
                mma_ss(tmX, desc_mn(vA, ks * 8, HALF32), desc_mn(uakA, ks * 8, HALF32), idesc64(32, 1, 1), 1, lead);
            cs.sync(lead);
            issue_solve(tmSA, tmX, d0A, n1A, lead, cs, [&]() {   // SA = Z T; meanwhile the parts of Y and S that do not need SA
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   // Y = X_r + V U_kr
                    mma_ss(tmX + 32, desc_mn(vA, ks * 8, HALF32), desc_mn(ukrA, ks * 8, HALF32), idesc64(32, 1, 1), 1, lead);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   // S += V K~
                    mma_ss(tmS, desc_mn(vA, ks * 8, HALF32), desc_mn(bkA + 32 * 128, ks * 8, HALF64), idesc64(64, 1, 1), 1, lead);
            });
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // Y += SA U_br
                mma_ts(tmX + 32, tmSA + ks * 8, desc_mn(ubrA, ks * 8, HALF32), idesc64(32, 0, 1), 1, lead);
            mma_commit(bar + 1, lead);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // S += SA B~
                mma_ts(tmS, tmSA + ks * 8, desc_mn(bkA, ks * 8, HALF64), idesc64(64, 0, 1), 1, lead);
            mma_commit(bar + 2, lead);
            if (cs.fail) fail = 4;
        }
        if (c + 1 < nchunks) fetch_chunk<6, FTPW>(raw, src, tok0, C, c + 1, T, warp, lane);   // under the chain
        WKV7_PHASE(6);   // issue of the chain, request of the next chunk
        // ---- 5. y out, state scaled -------------------------------------------------------------------
        if (!mbar_wait(bar + 1, par)) fail = 2;
        tc_fence_after();
        WKV7_PHASE(7);   // wait for Y
        {
            float Y[4][4];
            tmem_ld_tiles<4>(Y, tmX + 32 + lane_off);
            tmem_wait_ld();
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                    ystage[tt * 72 + i] = __float2bfloat16_rn(Y[nt][e]);
                }
        }
        __syncthreads();
        {
            const int tt = tid >> 2, seg = tid & 3;   // token, 16 channels
            if (tt < valid) {
                const uint4* sp = reinterpret_cast<const uint4*>(ystage + tt * 72 + seg * 16);
                uint4* dp = reinterpret_cast<uint4*>(y_ + tok0 + (i64)(c * LC + tt) * C + seg * 16);
                dp[0] = sp[0];
                dp[1] = sp[1];
            }
        }
        WKV7_PHASE(8);   // y to global
        if (!mbar_wait(bar + 2, par)) fail = 3;
        tc_fence_after();
        WKV7_PHASE(9);   // wait for the state update
        {
            float* dst = (c + 1 < nchunks) ? (ck ? ck + (i64)(c + 1) * 64 * 64 : nullptr) : (sT_ ? sT_ + sbase : nullptr);
            float Sd[8][4];
            tmem_ld_tiles<8>(Sd, tmS + lane_off);
            tmem_wait_ld();
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float2 we = *reinterpret_cast<const float2*>(We + nt * 8 + 2 * t);
                Sd[nt][0] *= we.x; Sd[nt][1] *= we.y; Sd[nt][2] *= we.x; Sd[nt][3] *= we.y;
                if (dst != nullptr) {
                    *reinterpret_cast<float2*>(dst + (row0 + g) * 64 + nt * 8 + 2 * t) = make_float2(Sd[nt][0], Sd[nt][1]);
                    *reinterpret_cast<float2*>(dst + (row0 + g + 8) * 64 + nt * 8 + 2 * t) = make_float2(Sd[nt][2], Sd[nt][3]);
                }
            }
            tmem_st_tiles<8>(tmS + lane_off, Sd);
            tmem_wait_st();
        }
        WKV7_PHASE(10);  // decay scaling, saved state
    }

    if (fail && tid == 0) {   // a wait ran out: record it and poison this unit's outputs so that they cannot pass as results
        atomicMax(&g_l32_fwd_error, fail);
        y_[tok0] = __ushort_as_bfloat16((unsigned short)0x7fc0);
        if (sT_ != nullptr) sT_[sbase] = __int_as_float(0x7fc00000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(tmS) : "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 32;" ::"r"(tmSA) : "memory");
    }
}

WKV7_PHASE_READER(rwkvb200_phase_clocks_l32_fwd)

}  // namespace v7x

int wkv7_l32_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k, const void* v,
                     const void* a, const void* b, void* y, float* sT, float* s, int test_expire, cudaStream_t st) {
    using namespace v7x;
    cudaError_t e = cudaFuncSetAttribute(wkv7x_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_forward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7x_forward_kernel<<<grid, FNT, FwdSmem::kBytes, st>>>(T, H, s0, (const bf16*)r, (const bf16*)w, (const bf16*)k,
                                                            (const bf16*)v, (const bf16*)a, (const bf16*)b, (bf16*)y, sT, s, test_expire);
    return check_launch("wkv7_forward(tcgen05, 32-token chunks)");
}

int wkv7_l32_bwd_error_clear();
int wkv7_l32_clear_errors() {
    const int z = 0;
    if (cudaMemcpyToSymbol(v7x::g_l32_fwd_error, &z, sizeof(int)) != cudaSuccess) return -1;
    return wkv7_l32_bwd_error_clear();
}

int wkv7_l32_fwd_error() {
    int h = 0;
    if (cudaMemcpyFromSymbol(&h, v7x::g_l32_fwd_error, sizeof(int)) != cudaSuccess) return -1;
    return h;
}

}  // namespace rwkvb200
