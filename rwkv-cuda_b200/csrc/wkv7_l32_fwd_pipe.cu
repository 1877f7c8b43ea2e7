// RWKV-7 forward, head size 64, bf16 activations, 32-token chunks on tcgen05: the two-stage form.
//
// Same algorithm and the same products as wkv7_l32_fwd.cu, split over two groups of 4 warps that work on
// consecutive chunks at the same time:
//   front group, chunk c+1: operand preparation, U, the masked matrices and the block inverses
//                           (nothing of it needs the carried state);
//   back group, chunk c:    the dependent chain X, Z, SA, Y and the state update, y out, decay scaling.
// Two sets of operand arrays are handed over through mbarriers (full / empty); inside a group the warps
// synchronise on a named barrier.  One thread block per SM (133 KB of shared memory, 256 columns of
// tensor memory); chosen for launches with at most one (batch, head) unit per SM, where the time is one
// unit's chain of chunks.
#include "wkv7_l32.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7q {

using namespace v7x;

constexpr int GNT = 128;          // threads per group
constexpr int PNT = 2 * GNT;

struct SetSmem {
    static constexpr int kAR = 0;
    static constexpr int kBK = kAR + ARR64;
    static constexpr int kV = kBK + ARR64;
    static constexpr int kUak = kV + ARR32;
    static constexpr int kUbr = kUak + HALF32;
    static constexpr int kUkr = kUbr + HALF32;
    static constexpr int kD0 = kUkr + HALF32;
    static constexpr int kN1 = kD0 + HALF32;
    static constexpr int kUab = kN1 + HALF32;           // plain [32][UPITCH] (front group only)
    static constexpr int kWe = kUab + 32 * UPITCH * 4;
    static constexpr int kHs = kWe + 256;               // [4][64] (front group only)
    static constexpr int kBytes = (kHs + 1024 + 1023) / 1024 * 1024;
};
struct PipeSmem {
    static constexpr int kSet1 = SetSmem::kBytes;
    static constexpr int kY = 2 * SetSmem::kBytes;      // bf16 [32][72]
    static constexpr int kBar = kY + 32 * 72 * 2;       // 10 mbarriers, tmem slot, abort words
    static constexpr int kBytes = kBar + 128 + 1024;
};
static_assert(PipeSmem::kBar % 8 == 0 && PipeSmem::kBytes <= 232448, "layout");

__device__ int g_l32_fwdp_error = 0;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// mbarriers: 0-1 full[set], 2-3 empty[set]; front: 4 U; back: 5 Y, 6 S, 7 its chain
enum { kFull = 0, kEmpty = 2, kFU = 4, kBY = 5, kBS = 6, kBChain = 7, kNBar = 8 };

__global__ void __launch_bounds__(PNT, 1)
wkv7q_forward_kernel(int T, int H, const float* __restrict__ s0_, const bf16* __restrict__ r_,
                     const bf16* __restrict__ w_, const bf16* __restrict__ k_, const bf16* __restrict__ v_,
                     const bf16* __restrict__ a_, const bf16* __restrict__ b_, bf16* __restrict__ y_,
                     float* __restrict__ sT_, float* __restrict__ ck_) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    bf16* ystage = reinterpret_cast<bf16*>(smem + PipeSmem::kY);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + PipeSmem::kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + kNBar);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* gabort = abort_word + 1;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int grp = warp >> 2, wg = warp & 3, gtid = tid & (GNT - 1);
    const int row0 = wg * 16;
    const int C = H * 64;
    const i64 tok0 = (i64)bb * T * C + hh * 64;
    const i64 sbase = (i64)(bb * H + hh) * 64 * 64;
    const int nchunks = (T + LC - 1) / LC;
    float* ck = ck_ ? ck_ + (i64)(bb * H + hh) * (T / 16) * 64 * 64 : nullptr;
    const bf16* src[6] = {r_, w_, k_, v_, a_, b_};

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kNBar; ++i) mbar_init(bar + i);
        *abort_word = 0; gabort[0] = 0; gabort[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < 2 * HALF32 / 4; i += PNT) {   // D0 and N1 of both sets: the blocks never written stay zero
        reinterpret_cast<float*>(smem + SetSmem::kD0)[i] = 0.f;
        reinterpret_cast<float*>(smem + PipeSmem::kSet1 + SetSmem::kD0)[i] = 0.f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm0 = __shfl_sync(0xffffffffu, tmem_slot[0], 0);
    const uint32_t tmS = tm0, tmX = tm0 + 64, tmSA = tm0 + 128, tmU = tm0 + 192;
    const uint32_t lane_off = (uint32_t)(wg * 32) << 16;
    const uint32_t lead = elect_one();
    const int gbar = 1 + grp;
    int fail = 0;

    if (grp == 0) {
        // ================================ front group ======================================================
        RawChunk<6, 8> raw;
        fetch_chunk<6, 8>(raw, src, tok0, C, 0, T, wg, lane);
        uint32_t par = 0;
        for (int c = 0; c < nchunks; ++c, par ^= 1) {
            const int set = c & 1, valid = min(LC, T - c * LC);
            unsigned char* base = smem + set * PipeSmem::kSet1;
            unsigned char *AR = base + SetSmem::kAR, *BK = base + SetSmem::kBK, *Vs = base + SetSmem::kV;
            unsigned char *Uak = base + SetSmem::kUak, *Ubr = base + SetSmem::kUbr, *Ukr = base + SetSmem::kUkr;
            unsigned char *D0 = base + SetSmem::kD0, *N1 = base + SetSmem::kN1;
            float* Uab = reinterpret_cast<float*>(base + SetSmem::kUab);
            float* We = reinterpret_cast<float*>(base + SetSmem::kWe);
            float* Hs = reinterpret_cast<float*>(base + SetSmem::kHs);
            if (c >= 2 && !mbar_wait(bar + kEmpty + set, ((c >> 1) - 1) & 1)) fail = 30;   // the back group released this set
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[0] = *abort_word;
            group_sync(gbar, GNT);
            if (gabort[0]) break;
            prepare_operands<6, 8, 4>(raw, valid, AR, BK, Vs, HALF32, nullptr, 0, We, Hs, nullptr, wg, lane, gbar);
            proxy_fence();
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (wg == 0) {
                issue_u(tmU, smem_u32(AR), smem_u32(BK), lead);
                mma_commit(bar + kFU, lead);
            }
            if (c + 1 < nchunks) fetch_chunk<6, 8>(raw, src, tok0, C, c + 1, T, wg, lane);   // under U
            if (!mbar_wait(bar + kFU, par)) fail = 31;
            tc_fence_after();
            {
                float u[8][4];
                tmem_ld_tiles<8>(u, tmU + lane_off);
                tmem_wait_ld();
                scatter_u(u, wg, lane, Uab, N1, Uak, Ubr, Ukr);
            }
            tc_fence_before();
            group_sync(gbar, GNT);
            if (wg < 2) tri_inverse16<UPITCH>(Uab + 16 * wg * (UPITCH + 1), D0, 16 * wg, lane);
            proxy_fence();
            group_sync(gbar, GNT);
            if (gtid == 0) mbar_arrive(bar + kFull + set);   // the set is complete
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
    } else {
        // ================================ back group =======================================================
        {   // initial state -> tensor memory (and saved as the start state of chunk 0)
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
        ChainSync cs{bar + kBChain, 0, 0};
        uint32_t par = 0;
        for (int c = 0; c < nchunks; ++c, par ^= 1) {
            const int set = c & 1, valid = min(LC, T - c * LC);
            unsigned char* base = smem + set * PipeSmem::kSet1;
            const float* We = reinterpret_cast<const float*>(base + SetSmem::kWe);
            const uint32_t arA = smem_u32(base + SetSmem::kAR), bkA = smem_u32(base + SetSmem::kBK), vA = smem_u32(base + SetSmem::kV);
            const uint32_t uakA = smem_u32(base + SetSmem::kUak), ubrA = smem_u32(base + SetSmem::kUbr), ukrA = smem_u32(base + SetSmem::kUkr);
            const uint32_t d0A = smem_u32(base + SetSmem::kD0), n1A = smem_u32(base + SetSmem::kN1);
            if (!mbar_wait(bar + kFull + set, (c >> 1) & 1)) fail = 40;   // the front group has filled this set
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[1] = *abort_word;
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (gabort[1]) break;
            if (wg == 0) {
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
                mma_commit(bar + kBY, lead);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   // S += SA B~
                    mma_ts(tmS, tmSA + ks * 8, desc_mn(bkA, ks * 8, HALF64), idesc64(64, 0, 1), 1, lead);
                mma_commit(bar + kBS, lead);
                if (cs.fail) fail = 41;
            }
            if (!mbar_wait(bar + kBY, par)) fail = 42;
            tc_fence_after();
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
            group_sync(gbar, GNT);
            {
                const int tt = gtid >> 2, seg = gtid & 3;   // token, 16 channels
                if (tt < valid) {
                    const uint4* sp = reinterpret_cast<const uint4*>(ystage + tt * 72 + seg * 16);
                    uint4* dp = reinterpret_cast<uint4*>(y_ + tok0 + (i64)(c * LC + tt) * C + seg * 16);
                    dp[0] = sp[0];
                    dp[1] = sp[1];
                }
            }
            if (!mbar_wait(bar + kBS, par)) fail = 43;
            tc_fence_after();
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
            tc_fence_before();
            group_sync(gbar, GNT);
            if (gtid == 0) mbar_arrive(bar + kEmpty + set);   // the front group may refill this set
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
    }

    tc_fence_before();
    __syncthreads();
    const int ab = *abort_word;
    if (ab && tid == 0) atomicMax(&g_l32_fwdp_error, ab);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tm0) : "memory");
}

}  // namespace v7q

int wkv7_l32_forward_pipelined(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k, const void* v,
                               const void* a, const void* b, void* y, float* sT, float* s, cudaStream_t st) {
    using namespace v7q;
    cudaError_t e = cudaFuncSetAttribute(wkv7q_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PipeSmem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_forward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7q_forward_kernel<<<grid, PNT, PipeSmem::kBytes, st>>>(T, H, s0, (const bf16*)r, (const bf16*)w, (const bf16*)k,
                                                             (const bf16*)v, (const bf16*)a, (const bf16*)b, (bf16*)y, sT, s);
    return check_launch("wkv7_forward(tcgen05, 32-token chunks, two stages)");
}

int wkv7_l32_fwdp_error(int clear) {
    int h = 0;
    if (clear) return cudaMemcpyToSymbol(v7q::g_l32_fwdp_error, &h, sizeof(int)) == cudaSuccess ? 0 : -1;
    if (cudaMemcpyFromSymbol(&h, v7q::g_l32_fwdp_error, sizeof(int)) != cudaSuccess) return -1;
    return h;
}

}  // namespace rwkvb200
