// RWKV-7 forward, head size 64, bf16 activations, 32-token chunks on tcgen05: the staged form.
//
// Same algorithm and the same products as wkv7_l32_fwd.cu, split over three groups of 4 warps that work on
// consecutive chunks at the same time:
//   loader group, chunk c+2:  the raw rows of the six input tensors arrive as tiled bulk copies (TMA, one
//                             [32 tokens][64 channels] tile per tensor and chunk, two chunks ahead); operand
//                             preparation ([A~;R~], [B~;K~], V, chunk decay);
//   matrix group, chunk c+1:  U on the tensor core, the masked matrices and the block inverses
//                             (nothing of either group needs the carried state);
//   chain group, chunk c:     the dependent chain X, Z, SA, Y and the state update, y out, decay scaling.
// Three sets of operand arrays and two sets of token x token matrices are handed on through mbarriers
// (full / empty; an operand set is released by the matrix group and by the chain group); inside a group the
// warps synchronise on a named barrier.  A thirteenth warp issues the bulk copies (a lane of the loader group pays
// about 55 cycles per copy; with the warp of its own B = 16, T = 4096 goes from 1.715 to 1.697 ms).  One thread block per SM (220 KB of shared memory, 256 columns of
// tensor memory).  Measured per chunk: loader 3.7 k cycles, matrix group 3.1 k, chain group 3.4 k, against
// 7.2 k for one thread block of wkv7_l32_fwd.cu alone and 11 k with three on an SM (3.7 k per chunk and SM):
// B = 16, T = 4096 1.70 ms against 1.94 ms, B = 2 0.27 ms against 0.48 ms.  What did not help: the 192 rows of
// a chunk as untiled bulk copies of 128 bytes (the copy engine takes about 60 cycles per copy: 13 k cycles per
// chunk), the chunk after next requested with plain loads into a second register set (the 48 loads take
// 1.7 k cycles to issue), eight loader warps (preparation 3.9 k instead of 3.3 k), the six tiles issued by
// six lanes instead of one, two loader groups on alternate chunks (16 warps: every group then waits on another,
// 4.0 k cycles per chunk; a third set of matrices to decouple them does not fit the shared memory).
#include <cuda.h>

#include "wkv7_l32.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
// Optional cycle counters of the groups (-DRWKVB200_PHASE_CLOCKS): group g uses phases 5g .. 5g+4
#ifdef RWKVB200_PHASE_CLOCKS
#define PIPE_MARK(k)                                                                                       \
    do {                                                                                                   \
        if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0) {                                             \
            const long long now_ = clock64();                                                              \
            atomicAdd(&g_phase_clocks[wg][(k) + 5 * grp], (unsigned long long)(now_ - pipe_last_));        \
            pipe_last_ = now_;                                                                             \
        }                                                                                                  \
    } while (0)
#else
#define PIPE_MARK(k)
#endif

namespace v7q {

using namespace v7x;

constexpr int GNT = 128;          // threads per group
constexpr int PNT = 3 * GNT + 32;   // three groups and the warp that issues the bulk copies
constexpr int NA = 3;             // operand sets in flight
constexpr int NU = 2;             // matrix sets in flight
constexpr int NS = 2;             // chunks of raw input rows in flight (bulk copies)

struct PipeSmem {
    static constexpr int kASet = 2 * ARR64 + ARR32;     // [A~;R~], [B~;K~], V
    static constexpr int kUSet = 5 * HALF32;            // U_ak, U_br, U_kr, D0, N1
    static constexpr int kU = NA * kASet;
    static constexpr int kWe = kU + NU * kUSet;         // chunk decay, one row of 64 floats per operand set
    static constexpr int kHs = kWe + NA * 256;          // [4][64] scratch of the loader group
    static constexpr int kUab = kHs + 1024;             // plain [32][UPITCH], scratch of the matrix group
    static constexpr int kY = kUab + 32 * UPITCH * 4;   // bf16 [32][72]
    static constexpr int kRaw = (kY + 32 * 72 * 2 + 127) / 128 * 128;   // raw input rows: [NS][6 tensors][32 tokens][64 bf16]
    static constexpr int kBar = kRaw + NS * 6 * 32 * 128;         // mbarriers, tmem slot, abort words
    static constexpr int kBytes = kBar + 256 + 1024;
};
static_assert(PipeSmem::kASet % 1024 == 0 && PipeSmem::kUSet % 1024 == 0 && PipeSmem::kBytes <= 232448, "layout");

__device__ int g_l32_fwdp_error = 0;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One [32 tokens][64 channels] bf16 tile of a (B*T, C) tensor -> shared memory (plain rows of 128 bytes) by the
// copy engine; x = first channel (a multiple of 8), y = first row; completion is counted in bytes on the mbarrier.
__device__ __forceinline__ void tma_tile(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
struct InputMaps {
    CUtensorMap m[6];   // r, w, k, v, a, b as (B*T, C) bf16, box 64 x 32
};
__device__ __forceinline__ void mbar_init_count(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// mbarriers: operand set full (loader -> matrix group) / empty (two arrivals: matrix and chain group);
// matrix set full (matrix -> chain group; it implies the operand set) / empty; U done; Y, S done; the chain's own;
// the raw rows of a stage have landed / have been taken into registers by the loader group (loader -> issuing warp)
enum { kFullA = 0, kEmptyA = kFullA + NA, kFullU = kEmptyA + NA, kEmptyU = kFullU + NU, kFU = kEmptyU + NU, kBY, kBS, kBChain,
       kRawFull, kTaken = kRawFull + NS, kNBar = kTaken + NS };

__global__ void __launch_bounds__(PNT, 1)
wkv7q_forward_kernel(int T, int H, const float* __restrict__ s0_, const __grid_constant__ InputMaps maps, bf16* __restrict__ y_,
                     float* __restrict__ sT_, float* __restrict__ ck_) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    bf16* ystage = reinterpret_cast<bf16*>(smem + PipeSmem::kY);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + PipeSmem::kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + kNBar);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* gabort = abort_word + 1;   // one copy per group, so that a group takes its decision on one value

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

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kNBar; ++i) mbar_init_count(bar + i, (i >= kEmptyA && i < kEmptyA + NA) ? 2 : 1);
        *abort_word = 0; gabort[0] = 0; gabort[1] = 0; gabort[2] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < NU * 2 * HALF32 / 4; i += PNT) {   // D0 and N1 of every matrix set: the blocks never written stay zero
        const int u = i / (2 * HALF32 / 4), j = i % (2 * HALF32 / 4);
        reinterpret_cast<float*>(smem + PipeSmem::kU + u * PipeSmem::kUSet + 3 * HALF32)[j] = 0.f;
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
#ifdef RWKVB200_PHASE_CLOCKS
    long long pipe_last_ = clock64();
#endif

    if (grp == 0) {
        // ================================ loader group =====================================================
        float* Hs = reinterpret_cast<float*>(smem + PipeSmem::kHs);
        // The raw rows of a chunk (6 tensors x 32 tokens x 128 bytes) come in as six tiled bulk copies (TMA), issued
        // by the thirteenth warp two chunks ahead and counted on an mbarrier; every thread then takes its part (a channel
        // pair of 8 tokens per tensor) into registers.  Rows beyond the sequence belong to the next batch row or
        // lie outside the tensor (read as zeros); they are masked when the registers are filled.
        unsigned char* stg = smem + PipeSmem::kRaw;
        int sa = 0, ua = 0;   // operand set of this chunk, how often it has been used before
        int c = 0;
        for (; c < nchunks; ++c) {
            const int valid = min(LC, T - c * LC), st = c & 1;
            unsigned char* A = smem + sa * PipeSmem::kASet;
            float* We = reinterpret_cast<float*>(smem + PipeSmem::kWe + sa * 256);
            PIPE_MARK(2);
            if (!mbar_wait(bar + kRawFull + st, (c >> 1) & 1)) fail = 31;                 // the rows have arrived
            if (ua >= 1 && !mbar_wait(bar + kEmptyA + sa, (ua - 1) & 1)) fail = 30;       // both consumers released this set
            PIPE_MARK(0);
            RawChunk<6, 8> raw;
#pragma unroll
            for (int x = 0; x < 6; ++x)
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int tt = 8 * wg + q;
                    raw.x[x][q] = tt < valid ? *reinterpret_cast<const uint32_t*>(stg + ((st * 6 + x) * 32 + tt) * 128 + 4 * lane) : 0u;
                }
            PIPE_MARK(3);
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[0] = *abort_word;
            group_sync(gbar, GNT);
            if (gtid == 0) mbar_arrive(bar + kTaken + st);   // every thread has taken its part of the rows: the stage may be refilled
            if (gabort[0]) break;
            PIPE_MARK(4);
            prepare_operands<6, 8, 4>(raw, valid, A, A + ARR64, A + 2 * ARR64, HALF32, nullptr, 0, We, Hs, nullptr, wg, lane, gbar);
            proxy_fence();
            group_sync(gbar, GNT);
            if (gtid == 0) mbar_arrive(bar + kFullA + sa);
            PIPE_MARK(1);
            if (++sa == NA) { sa = 0; ++ua; }
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
    } else if (grp == 1) {
        // ================================ matrix group =====================================================
        float* Uab = reinterpret_cast<float*>(smem + PipeSmem::kUab);
        int sa = 0, ua = 0;
        uint32_t par = 0;
        for (int c = 0; c < nchunks; ++c, par ^= 1) {
            const int su = c & 1;
            unsigned char* A = smem + sa * PipeSmem::kASet;
            unsigned char* U = smem + PipeSmem::kU + su * PipeSmem::kUSet;
            unsigned char *Uak = U, *Ubr = U + HALF32, *Ukr = U + 2 * HALF32, *D0 = U + 3 * HALF32, *N1 = U + 4 * HALF32;
            PIPE_MARK(4);
            if (!mbar_wait(bar + kFullA + sa, ua & 1)) fail = 35;                              // operands of this chunk
            if (c >= NU && !mbar_wait(bar + kEmptyU + su, ((c >> 1) - 1) & 1)) fail = 36;      // the chain group released this matrix set
            PIPE_MARK(0);
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[1] = *abort_word;
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (gabort[1]) break;
            if (wg == 0) {
                issue_u(tmU, smem_u32(A), smem_u32(A + ARR64), lead);
                mma_commit(bar + kFU, lead);
            }
            if (!mbar_wait(bar + kFU, par)) fail = 37;
            tc_fence_after();
            if (gtid == 0) mbar_arrive(bar + kEmptyA + sa);   // this group is done with the operand set
            PIPE_MARK(1);
            {
                float u[8][4];
                tmem_ld_tiles<8>(u, tmU + lane_off);
                tmem_wait_ld();
                scatter_u(u, wg, lane, Uab, N1, Uak, Ubr, Ukr);
            }
            tc_fence_before();
            group_sync(gbar, GNT);
            PIPE_MARK(2);
            if (wg < 2) tri_inverse16<UPITCH>(Uab + 16 * wg * (UPITCH + 1), D0, 16 * wg, lane);
            proxy_fence();
            group_sync(gbar, GNT);
            if (gtid == 0) mbar_arrive(bar + kFullU + su);   // the matrix set is complete
            PIPE_MARK(3);
            if (++sa == NA) { sa = 0; ++ua; }
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
    } else if (grp == 3) {
        // ================================ the warp that issues the bulk copies ==============================
        // One lane asks for the six tiles of a chunk, NS chunks ahead, as soon as the loader group has taken the
        // chunk that held the stage before (an issue costs a thread about 55 cycles: too much for the loader's lanes).
        if (lane == 0) {
            unsigned char* stg = smem + PipeSmem::kRaw;
            int c = 0;
            for (; c < nchunks; ++c) {
                const int st = c & 1;
                if (c >= NS && !mbar_wait(bar + kTaken + st, ((c >> 1) - 1) & 1)) { fail = 32; break; }
                if (*abort_word) break;
                uint64_t* fb = bar + kRawFull + st;
                mbar_expect_tx(fb, 6 * 32 * 128);
#pragma unroll
                for (int x = 0; x < 6; ++x) tma_tile(stg + (st * 6 + x) * 32 * 128, &maps.m[x], hh * 64, bb * T + c * LC, fb);
            }
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            // leaving early: the copies that are still in flight must have landed before the block may end
            if (*abort_word)
                for (int cc = max(0, c - NS); cc < c; ++cc) mbar_wait(bar + kRawFull + (cc & 1), (cc >> 1) & 1);
        }
    } else {
        // ================================ chain group ======================================================
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
        int sa = 0;
        uint32_t par = 0;
        for (int c = 0; c < nchunks; ++c, par ^= 1) {
            const int su = c & 1, valid = min(LC, T - c * LC);
            unsigned char* A = smem + sa * PipeSmem::kASet;
            unsigned char* U = smem + PipeSmem::kU + su * PipeSmem::kUSet;
            const float* We = reinterpret_cast<const float*>(smem + PipeSmem::kWe + sa * 256);
            const uint32_t arA = smem_u32(A), bkA = smem_u32(A + ARR64), vA = smem_u32(A + 2 * ARR64);
            const uint32_t uakA = smem_u32(U), ubrA = smem_u32(U + HALF32), ukrA = smem_u32(U + 2 * HALF32);
            const uint32_t d0A = smem_u32(U + 3 * HALF32), n1A = smem_u32(U + 4 * HALF32);
            PIPE_MARK(4);
            if (!mbar_wait(bar + kFullU + su, (c >> 1) & 1)) fail = 40;   // matrices (and with them the operands) of this chunk
            PIPE_MARK(0);
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[2] = *abort_word;
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (gabort[2]) break;
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
            PIPE_MARK(1);
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
            PIPE_MARK(2);
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
            if (gtid == 0) {   // the other groups may refill the sets
                mbar_arrive(bar + kEmptyA + sa);
                mbar_arrive(bar + kEmptyU + su);
            }
            PIPE_MARK(3);
            if (++sa == NA) sa = 0;
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
    }

    tc_fence_before();
    __syncthreads();
    const int ab = *abort_word;
    if (ab && tid == 0) {   // a wait ran out: record it and poison this unit's outputs so that they cannot pass as results
        atomicMax(&g_l32_fwdp_error, ab);
        y_[tok0] = __ushort_as_bfloat16((unsigned short)0x7fc0);
        if (sT_ != nullptr) sT_[sbase] = __int_as_float(0x7fc00000);
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tm0) : "memory");
}

WKV7_PHASE_READER(rwkvb200_phase_clocks_l32_fwdp)

}  // namespace v7q

namespace {
// cuTensorMapEncodeTiled through the runtime's driver entry point query (the library links the runtime only)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
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
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, 32};
    const cuuint32_t elem[2] = {1, 1};
    return encode_tiled()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

bool wkv7_make_tile_map(void* map, const void* base, unsigned long long rows, unsigned long long cols) {
    return encode_tiled() != nullptr && make_map(reinterpret_cast<CUtensorMap*>(map), base, rows, cols);
}

// Returns RWKVB200_OK, an error code, or 1 when tensor maps cannot be made here (no entry point in the driver, or a
// shape it refuses): the caller then uses the one-group kernel.
int wkv7_l32_forward_pipelined(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k, const void* v,
                               const void* a, const void* b, void* y, float* sT, float* s, cudaStream_t st) {
    using namespace v7q;
    if (encode_tiled() == nullptr) return 1;
    InputMaps maps;
    const void* in[6] = {r, w, k, v, a, b};
    for (int x = 0; x < 6; ++x)
        if (!make_map(&maps.m[x], in[x], (uint64_t)B * T, (uint64_t)H * 64)) return 1;
    cudaError_t e = cudaFuncSetAttribute(wkv7q_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PipeSmem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_forward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7q_forward_kernel<<<grid, PNT, PipeSmem::kBytes, st>>>(T, H, s0, maps, (bf16*)y, sT, s);
    return check_launch("wkv7_forward(tcgen05, 32-token chunks, three stages)");
}

int wkv7_l32_fwdp_error(int clear) {
    int h = 0;
    if (clear) return cudaMemcpyToSymbol(v7q::g_l32_fwdp_error, &h, sizeof(int)) == cudaSuccess ? 0 : -1;
    if (cudaMemcpyFromSymbol(&h, v7q::g_l32_fwdp_error, sizeof(int)) != cudaSuccess) return -1;
    return h;
}

}  // namespace rwkvb200
