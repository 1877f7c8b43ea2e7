// RWKV-6 / RWKV-5 forward, head size 64, bf16 activations, 32-token chunks on tcgen05: three warp groups on
// consecutive chunks, inputs by TMA (the structure of wkv7_l32_fwd_pipe.cu without the delta-rule terms).
//
// Per (batch, head), S indexed [value i][key j], d_t the decay of token t (per key channel):
//   y_t = S_{t-1} r_t + (sum_j r_t u k_t) v_t ;   S_t = S_{t-1} diag(d_t) + v_t k_t^T
// (wkv6/cuda/wkv6_cuda_v1.cu:15-66, wkv6_state/cuda/wkv6state_cuda_v1a.cu, wkv5_bf16/cuda/wkv5_cuda_v1b.cu:12-60
// of the reference project).  Within a chunk of L = 32 tokens let P_t = prod_{tau<=t} d_tau, P_{-1} = 1,
// We = P_31, and
//   r~_t = r_t P_{t-1}     k~_s = k_s / P_s     k^_s = u k_s / P_{s-1}
//   A[s,t] = k~_s . r~_t (s < t),   A[t,t] = k^_t . r~_t = sum_j r_t u k_t,   0 otherwise
// then with S0 the state at the start of the chunk and V = [v_t]:
//   Y = S0 R~^T + V A            S_end = (S0 + V K~) diag(We)
// All products are tcgen05.mma kind::tf32 (M = 64): the 64 x 32 product [K~;K^] R~^T gives the strict part
// of A in its rows 0-31 and the diagonal in the diagonal of its rows 32-63.  The divisions by P are safe while
// the summed |log d| of a chunk stays below 80; beyond that the kernel raises the flag of its (batch, head)
// unit and the general-shape kernel redoes that unit.
//
//   loader group, chunk c+2:  raw rows by TMA (r, k, v and a per-token decay input), operand preparation;
//   matrix group, chunk c+1:  [K~;K^] R~^T on the tensor core, A masked into shared memory;
//   chain group, chunk c:     X = S R~^T, Y = X + V A, S += V K~, y out, S scaled by We.
#include <cuda.h>

#include "wkv7_l32.cuh"
#include "wkv6_chunked.cuh"

namespace rwkvb200 {
namespace v6q {

using namespace v7x;

constexpr int GNT = 128;          // threads per group
constexpr int PNT = 3 * GNT;
constexpr int NA = 3;             // operand sets in flight
constexpr int NU = 2;             // A matrices in flight
constexpr int NS = 2;             // chunks of raw input rows in flight
constexpr int kRawStage = 3 * 4096 + 8192;   // r, k, v tiles (bf16) and the decay tile (bf16 or fp32)
constexpr float kMaxChunkLog2Decay = 80.f * 1.4426950408889634f;

struct Smem {
    static constexpr int kASet = ARR32 + ARR64 + ARR32;   // R~ [32][64], [K~;K^] [64][64], V [32][64]
    static constexpr int kU = NA * kASet;                 // A matrices, swizzled [32][32]
    static constexpr int kWe = kU + NU * HALF32;
    static constexpr int kHs = kWe + NA * 256;
    static constexpr int kY = kHs + 1024;                 // bf16 [32][72]
    static constexpr int kRaw = (kY + 32 * 72 * 2 + 127) / 128 * 128;
    static constexpr int kBar = kRaw + NS * kRawStage;
    static constexpr int kBytes = kBar + 256 + 1024;
};
static_assert(Smem::kASet % 1024 == 0 && Smem::kU % 1024 == 0 && Smem::kRaw % 128 == 0 && Smem::kBytes <= 232448, "layout");

__device__ int g_v6q_error = 0;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_tile(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void mbar_init_count(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

struct Maps {
    CUtensorMap m[4];   // r, k, v (B*T, C) bf16; the decay input (B*T, C) bf16 or fp32 (unused for a static decay)
};

enum { kFullA = 0, kEmptyA = kFullA + NA, kFullU = kEmptyA + NA, kEmptyU = kFullU + NU, kFU = kEmptyU + NU, kBY, kBS, kBChain,
       kRawFull, kNBar = kRawFull + NS };

// WMODE: 0 = fp32 log-decay (B,T,C), 1 = bf16 raw input (B,T,C) with log-decay = -exp(w), 2 = fp32 decay value (C),
// 3 = fp32 log-decay (C)   (the forms of wkv6_chunked.cu)
template <int WMODE>
__global__ void __launch_bounds__(PNT, 1)
wkv6q_forward_kernel(int T, int H, const __grid_constant__ Maps maps, const void* __restrict__ wstat_, const bf16* __restrict__ u_,
                     const void* __restrict__ s0_, int s0_kind, bf16* __restrict__ y_, float* __restrict__ sT_,
                     float* __restrict__ ck_, int* __restrict__ unsafe_, int flag_div) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    bf16* ystage = reinterpret_cast<bf16*>(smem + Smem::kY);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + Smem::kBar);
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
    constexpr bool kPerToken = WMODE < 2;
    float* ck = ck_ ? ck_ + (i64)(bb * H + hh) * nchunks * 64 * 64 : nullptr;   // chunk-start states for a backward pass
    const bool states_only = y_ == nullptr;                                  // no y: the pass that only saves the states
    constexpr int kWTile = WMODE == 0 ? 8192 : 4096;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kNBar; ++i) mbar_init_count(bar + i, (i >= kEmptyA && i < kEmptyA + NA) ? 2 : 1);
        *abort_word = 0; gabort[0] = 0; gabort[1] = 0; gabort[2] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm0 = __shfl_sync(0xffffffffu, tmem_slot[0], 0);
    const uint32_t tmS = tm0, tmX = tm0 + 64, tmU = tm0 + 96;
    const uint32_t lane_off = (uint32_t)(wg * 32) << 16;
    const uint32_t lead = elect_one();
    const int gbar = 1 + grp;
    int fail = 0;

    if (grp == 0) {
        // ================================ loader group =====================================================
        float* Hs = reinterpret_cast<float*>(smem + Smem::kHs);
        unsigned char* stg = smem + Smem::kRaw;
        const int j0 = 2 * lane;
        const float u0 = __bfloat162float(u_[hh * 64 + j0]), u1 = __bfloat162float(u_[hh * 64 + j0 + 1]);
        float ls0 = 0.f, ls1 = 0.f;   // log2 of a static decay
        if (WMODE == 2) {
            ls0 = __log2f(reinterpret_cast<const float*>(wstat_)[hh * 64 + j0]);
            ls1 = __log2f(reinterpret_cast<const float*>(wstat_)[hh * 64 + j0 + 1]);
        } else if (WMODE == 3) {
            ls0 = reinterpret_cast<const float*>(wstat_)[hh * 64 + j0] * 1.4426950408889634f;
            ls1 = reinterpret_cast<const float*>(wstat_)[hh * 64 + j0 + 1] * 1.4426950408889634f;
        }
        int issued = 0;
        auto issue_raw = [&](int c) {   // every warp's lane 0 issues its share of the tiles
            const int st = c & 1;
            uint64_t* fb = bar + kRawFull + st;
            if (lane == 0) {
                if (wg == 0) mbar_expect_tx(fb, 3 * 4096 + (kPerToken ? kWTile : 0));
                if (wg < 3) tma_tile(stg + st * kRawStage + wg * 4096, &maps.m[wg], hh * 64, bb * T + c * LC, fb);
                if (wg == 3 && kPerToken) tma_tile(stg + st * kRawStage + 3 * 4096, &maps.m[3], hh * 64, bb * T + c * LC, fb);
            }
            issued = c + 1;
        };
        issue_raw(0);
        if (nchunks > 1) issue_raw(1);
        int sa = 0, ua = 0;
        int c = 0;
        for (; c < nchunks; ++c) {
            const int valid = min(LC, T - c * LC), st = c & 1;
            unsigned char* A = smem + sa * Smem::kASet;
            unsigned char *RT = A, *KK = A + ARR32, *Vs = A + ARR32 + ARR64;
            float* We = reinterpret_cast<float*>(smem + Smem::kWe + sa * 256);
            if (!mbar_wait(bar + kRawFull + st, (c >> 1) & 1)) fail = 31;
            if (ua >= 1 && !mbar_wait(bar + kEmptyA + sa, (ua - 1) & 1)) fail = 30;
            // this thread: channels j0, j0+1 of tokens 8*wg .. 8*wg+7
            uint32_t xr[8], xk[8], xv[8];
            float ld0[8], ld1[8];   // log2 decay of the token
            const unsigned char* rs = stg + st * kRawStage;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int tt = 8 * wg + q;
                const bool in = tt < valid;
                xr[q] = in ? *reinterpret_cast<const uint32_t*>(rs + tt * 128 + 4 * lane) : 0u;
                xk[q] = in ? *reinterpret_cast<const uint32_t*>(rs + 4096 + tt * 128 + 4 * lane) : 0u;
                xv[q] = in ? *reinterpret_cast<const uint32_t*>(rs + 8192 + tt * 128 + 4 * lane) : 0u;
                if (WMODE == 1) {
                    const float2 w2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(rs + 12288 + tt * 128 + 4 * lane));
                    ld0[q] = in ? -fexp(w2.x) * 1.4426950408889634f : 0.f;
                    ld1[q] = in ? -fexp(w2.y) * 1.4426950408889634f : 0.f;
                } else if (WMODE == 0) {
                    const float2 w2 = *reinterpret_cast<const float2*>(rs + 12288 + tt * 256 + 8 * lane);
                    ld0[q] = in ? w2.x * 1.4426950408889634f : 0.f;
                    ld1[q] = in ? w2.y * 1.4426950408889634f : 0.f;
                } else {
                    ld0[q] = in ? ls0 : 0.f;
                    ld1[q] = in ? ls1 : 0.f;
                }
            }
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[0] = *abort_word;
            group_sync(gbar, GNT);   // (every thread has taken its part of the rows: the stage may be refilled)
            if (gabort[0]) break;
            if (c + NS < nchunks) issue_raw(c + NS);
            // cumulative log2 decays: within the warp's 8 tokens, then across the warps
            float cs0[8], cs1[8], run0 = 0.f, run1 = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) { run0 += ld0[q]; run1 += ld1[q]; cs0[q] = run0; cs1[q] = run1; }
            *reinterpret_cast<float2*>(Hs + wg * 64 + j0) = make_float2(run0, run1);
            group_sync(gbar, GNT);
            float base0 = 0.f, base1 = 0.f, tot0 = 0.f, tot1 = 0.f;
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
                const float2 h = *reinterpret_cast<const float2*>(Hs + gq * 64 + j0);
                if (gq < wg) { base0 += h.x; base1 += h.y; }
                tot0 += h.x; tot1 += h.y;
            }
            if (wg == 0) {
                *reinterpret_cast<float2*>(We + j0) = make_float2(fex2(tot0), fex2(tot1));
                if (-tot0 > kMaxChunkLog2Decay || -tot1 > kMaxChunkLog2Decay)   // this unit must be redone by the general-shape kernel
                    atomicOr(unsafe_ + (((bb / flag_div) * H + hh) & (kChunkedFlagUnits - 1)), 1);
            }
            float lp0 = base0, lp1 = base1;   // log2 P_{t-1}
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int tt = 8 * wg + q;
                // a chunk whose decay is beyond the bound is recomputed elsewhere: keep the values finite here
                const float l0 = fmaxf(base0 + cs0[q], -120.f), l1 = fmaxf(base1 + cs1[q], -120.f);
                const float p0 = fmaxf(lp0, -120.f), p1 = fmaxf(lp1, -120.f);
                const float wp0 = fex2(p0), wp1 = fex2(p1), iw0 = fex2(-l0), iw1 = fex2(-l1), ip0 = fex2(-p0), ip1 = fex2(-p1);
                const float2 r2 = bf16x2_to_f2(xr[q]), k2 = bf16x2_to_f2(xk[q]), v2 = bf16x2_to_f2(xv[q]);
                *reinterpret_cast<float2*>(RT + sw(tt, j0, HALF32)) = make_float2(tf32rf(r2.x * wp0), tf32rf(r2.y * wp1));
                *reinterpret_cast<float2*>(KK + sw(tt, j0, HALF64)) = make_float2(tf32rf(k2.x * iw0), tf32rf(k2.y * iw1));
                *reinterpret_cast<float2*>(KK + sw(32 + tt, j0, HALF64)) = make_float2(tf32rf(u0 * k2.x * ip0), tf32rf(u1 * k2.y * ip1));
                *reinterpret_cast<float2*>(Vs + sw(tt, j0, HALF32)) = v2;
                lp0 = base0 + cs0[q]; lp1 = base1 + cs1[q];
            }
            proxy_fence();
            group_sync(gbar, GNT);
            if (gtid == 0) mbar_arrive(bar + kFullA + sa);
            if (++sa == NA) { sa = 0; ++ua; }
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
        for (int cc = c; cc < issued; ++cc) mbar_wait(bar + kRawFull + (cc & 1), (cc >> 1) & 1);
    } else if (grp == 1) {
        // ================================ matrix group =====================================================
        int sa = 0, ua = 0;
        uint32_t par = 0;
        for (int c = 0; c < nchunks; ++c, par ^= 1) {
            const int su = c & 1;
            unsigned char* A = smem + sa * Smem::kASet;
            unsigned char* Am = smem + Smem::kU + su * HALF32;
            if (!mbar_wait(bar + kFullA + sa, ua & 1)) fail = 35;
            if (c >= NU && !mbar_wait(bar + kEmptyU + su, ((c >> 1) - 1) & 1)) fail = 36;
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[1] = *abort_word;
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (gabort[1]) break;
            if (states_only) {   // nothing to build: hand the sets on
                if (gtid == 0) { mbar_arrive(bar + kEmptyA + sa); mbar_arrive(bar + kFullU + su); }
                if (++sa == NA) { sa = 0; ++ua; }
                continue;
            }
            if (wg == 0) {   // [K~;K^] R~^T: rows 0-31 = k~_s, 32-63 = k^_s; columns = tokens t
                const uint32_t kkA = smem_u32(A + ARR32), rtA = smem_u32(A);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    mma_ss(tmU, desc_k(kkA, 0, ks * 8, HALF64), desc_k(rtA, 0, ks * 8, HALF32), idesc64(32, 0, 0), ks > 0, lead);
                mma_commit(bar + kFU, lead);
            }
            if (!mbar_wait(bar + kFU, par)) fail = 37;
            tc_fence_after();
            if (gtid == 0) mbar_arrive(bar + kEmptyA + sa);   // this group is done with the operand set
            {
                float u[4][4];
                tmem_ld_tiles<4>(u, tmU + lane_off);
                tmem_wait_ld();
                const int sb = 16 * (wg & 1) + g;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int s = sb + 8 * h, c0 = nt * 8 + 2 * t;
                        if (wg < 2) {   // strict part; the diagonal comes from the other two warps
                            float* p = reinterpret_cast<float*>(Am + sw32(s, c0));
                            if (s != c0) p[0] = s < c0 ? tf32rf(u[nt][2 * h]) : 0.f;
                            if (s != c0 + 1) p[1] = s < c0 + 1 ? tf32rf(u[nt][2 * h + 1]) : 0.f;
                        } else {        // rows 32+s: the diagonal
                            float* p = reinterpret_cast<float*>(Am + sw32(s, c0));
                            if (s == c0) p[0] = tf32rf(u[nt][2 * h]);
                            if (s == c0 + 1) p[1] = tf32rf(u[nt][2 * h + 1]);
                        }
                    }
            }
            proxy_fence();
            tc_fence_before();
            group_sync(gbar, GNT);
            if (gtid == 0) mbar_arrive(bar + kFullU + su);
            if (++sa == NA) { sa = 0; ++ua; }
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
    } else {
        // ================================ chain group ======================================================
        {   // initial state -> tensor memory
            float Sd[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const i64 idx = sbase + (row0 + g + ((e & 2) ? 8 : 0)) * 64 + nt * 8 + 2 * t + (e & 1);
                    Sd[nt][e] = s0_kind == 2 ? reinterpret_cast<const float*>(s0_)[idx]
                              : s0_kind == 1 ? __bfloat162float(reinterpret_cast<const bf16*>(s0_)[idx]) : 0.f;
                }
            if (ck != nullptr) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    *reinterpret_cast<float2*>(ck + (row0 + g) * 64 + nt * 8 + 2 * t) = make_float2(Sd[nt][0], Sd[nt][1]);
                    *reinterpret_cast<float2*>(ck + (row0 + g + 8) * 64 + nt * 8 + 2 * t) = make_float2(Sd[nt][2], Sd[nt][3]);
                }
            }
            tmem_st_tiles<8>(tmS + lane_off, Sd);
            tmem_wait_st();
        }
        ChainSync cs{bar + kBChain, 0, 0};
        int sa = 0;
        uint32_t par = 0;
        for (int c = 0; c < nchunks; ++c, par ^= 1) {
            const int su = c & 1, valid = min(LC, T - c * LC);
            unsigned char* A = smem + sa * Smem::kASet;
            const float* We = reinterpret_cast<const float*>(smem + Smem::kWe + sa * 256);
            const uint32_t rtA = smem_u32(A), kkA = smem_u32(A + ARR32), vA = smem_u32(A + ARR32 + ARR64);
            const uint32_t amA = smem_u32(smem + Smem::kU + su * HALF32);
            if (!mbar_wait(bar + kFullU + su, (c >> 1) & 1)) fail = 40;
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[2] = *abort_word;
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (gabort[2]) break;
            if (wg == 0) {
                if (!states_only) {
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)   // X = S R~^T
                        mma_ts(tmX, tmS + ks * 8, desc_k(rtA, 0, ks * 8, HALF32), idesc64(32, 0, 0), ks > 0, lead);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)   // Y = X + V A
                        mma_ss(tmX, desc_mn(vA, ks * 8, HALF32), desc_mn(amA, ks * 8, HALF32), idesc64(32, 1, 1), 1, lead);
                    mma_commit(bar + kBY, lead);
                    cs.sync(lead);                   // X has read S: it may be updated
                }
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   // S += V K~
                    mma_ss(tmS, desc_mn(vA, ks * 8, HALF32), desc_mn(kkA, ks * 8, HALF64), idesc64(64, 1, 1), 1, lead);
                mma_commit(bar + kBS, lead);
                if (cs.fail) fail = 41;
            }
            if (!states_only && !mbar_wait(bar + kBY, par)) fail = 42;
            tc_fence_after();
            if (!states_only) {
                float Y[4][4];
                tmem_ld_tiles<4>(Y, tmX + lane_off);
                tmem_wait_ld();
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                        ystage[tt * 72 + i] = __float2bfloat16_rn(Y[nt][e]);
                    }
            }
            tc_fence_before();
            group_sync(gbar, GNT);
            if (!states_only) {
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
            if (gtid == 0) {
                mbar_arrive(bar + kEmptyA + sa);
                mbar_arrive(bar + kEmptyU + su);
            }
            if (++sa == NA) sa = 0;
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
    }

    tc_fence_before();
    __syncthreads();
    const int ab = *abort_word;
    if (ab && tid == 0) {   // a wait ran out: record it and poison this unit's outputs
        atomicMax(&g_v6q_error, ab);
        if (y_ != nullptr) y_[tok0] = __ushort_as_bfloat16((unsigned short)0x7fc0);
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(tm0) : "memory");
}

}  // namespace v6q

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled6() {
    if (tensor_maps_disabled()) return nullptr;
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}
bool make_map6(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, bool fp32) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * (fp32 ? 4 : 2)};
    const cuuint32_t box[2] = {64, 32};
    const cuuint32_t elem[2] = {1, 1};
    return encode_tiled6()(m, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                           strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

bool wkv6_make_tile_map(void* map, const void* base, unsigned long long rows, unsigned long long cols, bool fp32) {
    return encode_tiled6() != nullptr && make_map6(reinterpret_cast<CUtensorMap*>(map), base, rows, cols, fp32);
}

// Returns RWKVB200_OK, an error code, or 1 when tensor maps cannot be made here (the caller then uses the
// mma.sync kernel of wkv6_chunked.cu).  Arguments as wkv6_chunked_forward; ck (optional): the states at the start of
// every 32-token chunk, (B,H,ceil(T/32),N,N) fp32, for wkv6_l32_backward; y may then be NULL (states only).
int wkv6_l32_forward(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode, const void* u,
                     const void* s0, int s0_kind, void* y, float* sT, float* ck, int* unsafe, cudaStream_t st, int flag_div) {
    using namespace v6q;
    if (encode_tiled6() == nullptr) return 1;
    Maps maps;
    const void* in[3] = {r, k, v};
    for (int x = 0; x < 3; ++x)
        if (!make_map6(&maps.m[x], in[x], (uint64_t)B * T, (uint64_t)H * 64, false)) return 1;
    if (w_mode < 2) {
        if (!make_map6(&maps.m[3], w, (uint64_t)B * T, (uint64_t)H * 64, w_mode == 0)) return 1;
    } else {
        maps.m[3] = maps.m[0];
    }
    dim3 grid(H, B);
#define RWKV_GO(M)                                                                                                       \
    do {                                                                                                                 \
        cudaError_t e = cudaFuncSetAttribute(wkv6q_forward_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes); \
        RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv6_forward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));  \
        wkv6q_forward_kernel<M><<<grid, PNT, Smem::kBytes, st>>>(T, H, maps, w, (const bf16*)u, s0, s0_kind, (bf16*)y, sT, \
                                                                ck, unsafe, flag_div);                                       \
    } while (0)
    switch (w_mode) {
        case 0: RWKV_GO(0); break;
        case 1: RWKV_GO(1); break;
        case 2: RWKV_GO(2); break;
        default: RWKV_GO(3); break;
    }
#undef RWKV_GO
    return check_launch("wkv6_forward(tcgen05, 32-token chunks, three stages)");
}

int wkv6_l32_error(int clear) {
    int h = 0;
    if (clear) return cudaMemcpyToSymbol(v6q::g_v6q_error, &h, sizeof(int)) == cudaSuccess ? 0 : -1;
    if (cudaMemcpyFromSymbol(&h, v6q::g_v6q_error, sizeof(int)) != cudaSuccess) return -1;
    return h;
}

}  // namespace rwkvb200
