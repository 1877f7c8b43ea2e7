// RWKV-7 backward, head size 64, bf16 activations, 32-token chunks on tcgen05: the two-stage form.
//
// Same algorithm and the same products as wkv7_l32_bwd.cu (results equal up to how the compiler fuses the
// last multiply-adds of the epilogue: a handful of dw elements differ by one bf16 ulp), split over two groups
// of 8 warps that work on consecutive chunks at the same time:
//   front group, chunk c-1: everything that does not need the carried state gradient -- operand
//       preparation, U, the masked matrices and the block inverses, the forward part again (SA);
//   back group, chunk c:    decay scaling of E / ET, EV and dV, P, the gradients of the scaled vectors,
//       the update of E / ET, the epilogue.
// Each stage takes about half of a chunk's time, so a lone thread block finishes a chunk in a little over
// half the time of the one-group kernel.  The price is a second set of operand arrays (222 KB of shared
// memory) and the whole tensor memory of the SM: one thread block per SM.  It is chosen for launches
// with at most one (batch, head) unit per SM, where the time is one unit's chain of chunks.
// The sets are handed over through two pairs of mbarriers (full / empty); inside a group the warps
// synchronise on a named barrier; each group has its own issuing warp and its own mbarriers.
#include "wkv7_l32.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
// Optional cycle counters of the two groups (-DRWKVB200_PHASE_CLOCKS): front group phases 0.., back group 8..
#ifdef RWKVB200_PHASE_CLOCKS
#define PIPE_MARK(k)                                                                                       \
    do {                                                                                                   \
        if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0) {                                             \
            const long long now_ = clock64();                                                              \
            atomicAdd(&g_phase_clocks[wg][(k) + 8 * grp], (unsigned long long)(now_ - pipe_last_));   \
            pipe_last_ = now_;                                                                             \
        }                                                                                                  \
    } while (0)
#else
#define PIPE_MARK(k)
#endif

namespace v7p {

using namespace v7x;

constexpr int GNT = 256;          // threads per group
constexpr int PNT = 2 * GNT;      // threads per CTA
constexpr int BPITCH = 20;

// one set of operands of a chunk
struct SetSmem {
    static constexpr int kAR = 0;
    static constexpr int kBK = kAR + ARR64;
    static constexpr int kSV = kBK + ARR64;              // rows 0-31 SA_t, rows 32-63 v_t
    static constexpr int kEY = kSV + ARR64;              // rows 0-31 EV_u, rows 32-63 dy_u
    static constexpr int kS0 = kEY + ARR64;              // [i][j]
    static constexpr int kUak = kS0 + ARR64;             // Uak Ubr Ukr D0: 4 x [32][32]; later P [64][64]
    static constexpr int kUbr = kUak + HALF32;
    static constexpr int kUkr = kUbr + HALF32;
    static constexpr int kD0 = kUkr + HALF32;
    static constexpr int kP = kUak;
    static constexpr int kN1 = kD0 + HALF32;
    static constexpr int kLam = kN1 + HALF32;            // plain [32][LAMP]
    static constexpr int kWe = kLam + 32 * LAMP * 4;     // [64]
    static constexpr int kBytes = (kWe + 256 + 1023) / 1024 * 1024;
    static constexpr int kHs = kEY;                      // scratch inside the EV rows (front group only)
    static constexpr int kUab = kEY + HALF64;
};
static_assert(SetSmem::kBytes % 1024 == 0, "sets start on 1024-byte boundaries");
struct PipeSmem {
    static constexpr int kSet1 = SetSmem::kBytes;
    static constexpr int kA0 = 2 * SetSmem::kBytes;      // [2][64]
    static constexpr int kCarry = kA0 + 512;             // [64]
    static constexpr int kBar = kCarry + 256;            // 15 mbarriers, tmem slot, abort words, request counters
    static constexpr int kBytes = kBar + 256 + 1024;
};
static_assert(PipeSmem::kBytes <= 232448, "fits the shared memory of one SM");

__device__ int g_l32_bwdp_error = 0;

// Tensors X0 .. X1-1 of a thread's part of chunk c (fetch_chunk in pieces: a burst of 28 four-byte loads per
// thread from all warps at once takes 1.3 k cycles to issue, so the pieces go where the warps would wait anyway).
template <int X0, int X1>
__device__ __forceinline__ void fetch_part(RawChunk<7, 4>& rc, const bf16* const* src, i64 tok0, int C, int c, int T, int warp, int lane) {
    const int t0 = c * LC + 4 * warp;
    const i64 off = tok0 + (i64)t0 * C + 2 * lane;
#pragma unroll
    for (int x = X0; x < X1; ++x)
#pragma unroll
        for (int q = 0; q < 4; ++q)
            rc.x[x][q] = (t0 + q < T) ? __ldg(reinterpret_cast<const unsigned int*>(src[x] + off + (i64)q * C)) : 0u;
}

__device__ __forceinline__ void scatter_u_half(const float (*u)[4], int quarter, int hs, int lane, float* Uab, unsigned char* N1,
                                               unsigned char* Uak, unsigned char* Ubr, unsigned char* Ukr) {
    const int g = lane >> 2, t = lane & 3;
    const int sb = 16 * (quarter & 1) + g;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int s = sb + 8 * h, c0 = nt * 8 + 2 * t;
            if (hs == 0) {
                const float a0 = s < c0 ? u[nt][2 * h] : 0.f, a1 = s < c0 + 1 ? u[nt][2 * h + 1] : 0.f;
                if (quarter < 2) {
                    if ((nt >> 1) == quarter) *reinterpret_cast<float2*>(Uab + (quarter * 16 + (s & 15)) * BPITCH + (c0 & 15)) = make_float2(a0, a1);
                    if (quarter == 0 && nt >= 2) *reinterpret_cast<float2*>(N1 + sw32(s, c0)) = make_float2(tf32rf(a0), tf32rf(a1));
                } else {
                    *reinterpret_cast<float2*>(Uak + sw32(s, c0)) = make_float2(tf32rf(a0), tf32rf(a1));
                }
            } else {
                const float r0 = s <= c0 ? u[nt][2 * h] : 0.f, r1 = s <= c0 + 1 ? u[nt][2 * h + 1] : 0.f;
                *reinterpret_cast<float2*>((quarter < 2 ? Ubr : Ukr) + sw32(s, c0)) = make_float2(tf32rf(r0), tf32rf(r1));
            }
        }
}

__device__ __forceinline__ float tf32_seen(const unsigned char* p) {
    return __uint_as_float(*reinterpret_cast<const uint32_t*>(p) & 0xffffe000u);
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// mbarriers: 0-1 full[set], 2-3 empty[set] (one arrival each); front: 4 U, 5-6 SA[set], 7 its chain; back: 8 EV,
// 9 P, 10 E/ET, 11 gradients, 12 its chain; 13-14 the staged input tiles of a set have landed
enum { kFull = 0, kEmpty = 2, kFU = 4, kFSA = 5, kFChain = 7, kBEV = 8, kBP = 9, kBE = 10, kBG = 11, kBChain = 12, kRaw = 13, kNBar = 15 };

__global__ void __launch_bounds__(PNT, 1)
wkv7p_backward_kernel(int T, int H, const bf16* __restrict__ r_, const bf16* __restrict__ w_,
                      const bf16* __restrict__ k_, const bf16* __restrict__ v_, const bf16* __restrict__ a_,
                      const bf16* __restrict__ b_, const bf16* __restrict__ dy_, const float* __restrict__ dsT_,
                      const float* __restrict__ ck_, float* __restrict__ ds0_, bf16* __restrict__ dr_,
                      bf16* __restrict__ dw_, bf16* __restrict__ dk_, bf16* __restrict__ dv_, bf16* __restrict__ da_,
                      bf16* __restrict__ db_, const __grid_constant__ TileMaps<7> maps) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    float* A0p = reinterpret_cast<float*>(smem + PipeSmem::kA0);
    float* Carry = reinterpret_cast<float*>(smem + PipeSmem::kCarry);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + PipeSmem::kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + kNBar);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* gabort = abort_word + 1;   // [2]: each group's copy, so that all its threads take the same decision
    volatile int* raw_req = gabort + 2;      // [2]: tile requests issued per set;  raw_got = raw_req + 2: [2] requests whose tiles were taken
    volatile int* raw_got = raw_req + 2;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int grp = warp >> 3, wg = warp & 7, gtid = tid & (GNT - 1);   // group, warp and thread inside the group
    const int quarter = wg & 3, hs = wg >> 2;
    const int row0 = quarter * 16;
    const int C = H * 64;
    const i64 tok0 = (i64)bb * T * C + hh * 64;
    const i64 sbase = (i64)(bb * H + hh) * 64 * 64;
    const int nchunks = (T + LC - 1) / LC;
    const float* ck = ck_ + (i64)(bb * H + hh) * (T / 16) * 64 * 64;
    const bf16* src[7] = {r_, w_, k_, v_, a_, b_, dy_};

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kNBar; ++i) mbar_init(bar + i);
        *abort_word = 0; gabort[0] = 0; gabort[1] = 0;
        raw_req[0] = raw_req[1] = raw_got[0] = raw_got[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < HALF32 / 4; i += PNT) {   // N1 of both sets: only the upper right block is ever written
        reinterpret_cast<float*>(smem + SetSmem::kN1)[i] = 0.f;
        reinterpret_cast<float*>(smem + PipeSmem::kSet1 + SetSmem::kN1)[i] = 0.f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm0 = __shfl_sync(0xffffffffu, tmem_slot[0], 0);
    const uint32_t tmE = tm0, tmET = tm0 + 64, tmW1 = tm0 + 128, tmW2 = tm0 + 192, tmF1 = tm0 + 256, tmF2a = tm0 + 320, tmF2b = tm0 + 384;   // X_a / SA per set
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t lead = elect_one();
    const int gbar = 1 + grp;   // named barrier of this group
    int fail = 0;
#ifdef RWKVB200_PHASE_CLOCKS
    long long pipe_last_ = clock64();
#endif

    // With tensor maps the inputs of a chunk come by the copy engine into EY and the first 12 KB of S0 of the set that
    // the chunk will use, as soon as the chunk that used the set before has no more use for them: asked for by one
    // thread of the back group after its last products (by the front group for the first two chunks), counted in
    // bytes on the set's mbarrier; the front group takes its words out of the tiles before it writes the set.
    const bool staged = maps.valid != 0;
    // (called by every thread of a group: lane 0 of the group's warp x asks for tile x, an issue costs a thread about
    // 55 cycles; warp 0 announces the bytes, which may happen before or after the other warps' copies complete)
    auto request = [&](int set, int c) {
        if (lane != 0) return;
        unsigned char* dst = smem + set * PipeSmem::kSet1 + SetSmem::kEY;
        if (wg == 0) {
            mbar_expect_bytes(bar + kRaw + set, 7 * 4096);
            raw_req[set] = raw_req[set] + 1;
        }
        if (wg < 7) tma_tile_load(dst + wg * 4096, &maps.m[wg], hh * 64, bb * T + c * LC, bar + kRaw + set);
    };

    // ================================ front group ==========================================================
    if (grp == 0) {
        RawChunk<7, 4> raw;
        if (!staged) fetch_chunk<7, 4>(raw, src, tok0, C, nchunks - 1, T, wg, lane);
        else {
            request(0, nchunks - 1);
            if (nchunks > 1) request(1, nchunks - 2);
        }
        ChainSync cs{bar + kFChain, 0, 0};   // used by the group's warp 0 only
        // dr, da, dk, db, dw of chunk cp, staged as bf16 rows by the back group in dead arrays of the set at
        // `sbase_`, go to global memory from this group (thread = token, 16-byte piece), which has the time.
        auto flush_outputs = [&](unsigned char* sbase_, int cp) {
            const int tt = gtid >> 3, piece = gtid & 7;
            if (tt < min(LC, T - cp * LC)) {
                const bf16* st0 = reinterpret_cast<const bf16*>(sbase_ + SetSmem::kSV) + tt * 72 + piece * 8;
                const bf16* st3 = reinterpret_cast<const bf16*>(sbase_ + SetSmem::kP) + tt * 72 + piece * 8;
                const i64 o = tok0 + (i64)(cp * LC + tt) * C + piece * 8;
                *reinterpret_cast<uint4*>(dr_ + o) = *reinterpret_cast<const uint4*>(st0);
                *reinterpret_cast<uint4*>(da_ + o) = *reinterpret_cast<const uint4*>(st0 + 32 * 72);
                *reinterpret_cast<uint4*>(dk_ + o) = *reinterpret_cast<const uint4*>(st0 + 2 * 32 * 72);
                *reinterpret_cast<uint4*>(db_ + o) = *reinterpret_cast<const uint4*>(st3);
                *reinterpret_cast<uint4*>(dw_ + o) = *reinterpret_cast<const uint4*>(st3 + 32 * 72);
            }
            stage_flush(sbase_ + SetSmem::kN1, dv_, tok0 + (i64)cp * LC * C, C, gtid, min(LC, T - cp * LC));
        };
        uint32_t par = 0;
        int it = 0;
        for (int c = nchunks - 1; c >= 0; --c, ++it, par ^= 1) {
            const int set = it & 1, valid = min(LC, T - c * LC);
            unsigned char* base = smem + set * PipeSmem::kSet1;
            unsigned char *AR = base + SetSmem::kAR, *BK = base + SetSmem::kBK, *SV = base + SetSmem::kSV, *EY = base + SetSmem::kEY;
            unsigned char *S0 = base + SetSmem::kS0, *Uak = base + SetSmem::kUak, *Ubr = base + SetSmem::kUbr, *Ukr = base + SetSmem::kUkr;
            unsigned char *D0 = base + SetSmem::kD0, *N1 = base + SetSmem::kN1;
            float* Lam = reinterpret_cast<float*>(base + SetSmem::kLam);
            float* We = reinterpret_cast<float*>(base + SetSmem::kWe);
            float* Hs = reinterpret_cast<float*>(base + SetSmem::kHs);
            float* Uab = reinterpret_cast<float*>(base + SetSmem::kUab);
            const uint32_t arA = smem_u32(AR), bkA = smem_u32(BK), svA = smem_u32(SV), s0A = smem_u32(S0);
            const uint32_t uakA = smem_u32(Uak), d0A = smem_u32(D0), n1A = smem_u32(N1);
            const uint32_t tmF2 = set ? tmF2b : tmF2a;
            // the back group must have released this set (it was used two chunks ago)
            PIPE_MARK(1);
            if (it >= 2 && !mbar_wait(bar + kEmpty + set, ((it >> 1) - 1) & 1)) fail = 30;
            PIPE_MARK(0);
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[0] = *abort_word;
            group_sync(gbar, GNT);
            if (gabort[0]) break;
            if (it >= 2) flush_outputs(base, c + 2);   // the set holds the staged outputs of the chunk that used it last: they leave from here
            if (staged) {
                if (!mbar_wait(bar + kRaw + set, (it >> 1) & 1)) fail = 36;
                const unsigned char* rawt = base + SetSmem::kEY;
#pragma unroll
                for (int x = 0; x < 7; ++x)
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        raw.x[x][q] = (c * LC + 4 * wg + q < T) ? *reinterpret_cast<const uint32_t*>(rawt + x * 4096 + (4 * wg + q) * 128 + lane * 4) : 0u;
                if (gtid == 0) raw_got[set] = raw_got[set] + 1;
            }
            if (it >= 2 || staged) group_sync(gbar, GNT);   // before the set is written
            {   // chunk-start state -> S0 (swizzled), 16-byte pieces
                const float* s0g = ck + (i64)c * 64 * 64;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int idx = q4 * GNT + gtid, i = idx >> 4, col = (idx & 15) * 4;
                    cp_async16(S0 + sw(i, col, HALF64), s0g + i * 64 + col);
                }
                cp_async_commit();
            }
            {   // the zero blocks of D0 (its space was used by P), and N1 (it held the staged dv; only its upper right
                // block is written below, the rest has to read as zero)
                const int s = gtid >> 4, cc = gtid & 15;
                *reinterpret_cast<float*>(D0 + sw32(s, 16 + cc)) = 0.f;
                *reinterpret_cast<float*>(D0 + sw32(16 + s, cc)) = 0.f;
                reinterpret_cast<float4*>(N1)[gtid] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            prepare_operands<7, 4, 8>(raw, valid, AR, BK, SV + 32 * 128, HALF64, EY + 32 * 128, HALF64, We, Hs, Lam, wg, lane, gbar);
            cp_async_wait<0>();
            proxy_fence();
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (wg == 0) {
                issue_u(tmF1, arA, bkA, lead);
                mma_commit(bar + kFU, lead);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   // X_a = S0 A~^T, needed after the inverse only
                    mma_ss(tmF2, desc_k(s0A, 0, ks * 8, HALF64), desc_k(arA, 0, ks * 8, HALF64), idesc64(32, 0, 0), ks > 0, lead);
            }
            if (c > 0 && !staged) fetch_part<0, 4>(raw, src, tok0, C, c - 1, T, wg, lane);   // the next chunk, first part: under U
            PIPE_MARK(2);
            if (!mbar_wait(bar + kFU, par)) fail = 31;
            PIPE_MARK(3);
            tc_fence_after();
            {
                float u[4][4];
                tmem_ld_tiles<4>(u, tmF1 + 32 * hs + lane_off);
                tmem_wait_ld();
                scatter_u_half(u, quarter, hs, lane, Uab, N1, Uak, Ubr, Ukr);
            }
            tc_fence_before();
            group_sync(gbar, GNT);
            PIPE_MARK(4);
            if (wg < 2) tri_inverse16<BPITCH>(Uab + wg * 16 * BPITCH, D0, 16 * wg, lane);
            proxy_fence();
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (wg == 0) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   // Z = X_a + V U_ak
                    mma_ss(tmF2, desc_mn(svA + 32 * 128, ks * 8, HALF64), desc_mn(uakA, ks * 8, HALF32), idesc64(32, 1, 1), 1, lead);
                cs.sync(lead);
                issue_solve(tmF2 + 32, tmF2, d0A, n1A, lead, cs, [&]() {   // SA = Z T
                    if (c > 0 && !staged) fetch_part<4, 7>(raw, src, tok0, C, c - 1, T, wg, lane);
                });
                mma_commit(bar + kFSA + set, lead);   // the back group takes SA out of tensor memory
                if (cs.fail) fail = 32;
            } else if (c > 0 && !staged) {
                fetch_part<4, 7>(raw, src, tok0, C, c - 1, T, wg, lane);   // the next chunk, second part: under the chain
            }
            PIPE_MARK(5);
            proxy_fence();
            tc_fence_before();
            group_sync(gbar, GNT);
            if (gtid == 0) mbar_arrive(bar + kFull + set);   // the set is complete (but for SA, which the back group converts)
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
        // the outputs of the last two chunks (iterations nchunks-2 and nchunks-1 of the back group)
        for (int j = max(0, nchunks - 2); j < nchunks && !fail; ++j) {
            if (!mbar_wait(bar + kEmpty + (j & 1), (j >> 1) & 1)) { fail = 34; atomicMax(const_cast<int*>(abort_word), fail); }
            if (gtid == 0) gabort[0] = *abort_word;
            group_sync(gbar, GNT);
            if (gabort[0]) break;
            flush_outputs(smem + (j & 1) * PipeSmem::kSet1, nchunks - 1 - j);
            group_sync(gbar, GNT);
        }
    }

    // ================================ back group ===========================================================
    if (grp == 1) {
        {   // E, ET <- dsT (or zero); this warp: its 16 rows, columns 32*hs .. 32*hs+31
            float Ed[4][4], Td[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = row0 + g + ((e & 2) ? 8 : 0), col = 32 * hs + nt * 8 + 2 * t + (e & 1);
                    Ed[nt][e] = dsT_ ? dsT_[sbase + row * 64 + col] : 0.f;
                    Td[nt][e] = dsT_ ? dsT_[sbase + col * 64 + row] : 0.f;
                }
            tmem_st_tiles<4>(tmE + 32 * hs + lane_off, Ed);
            tmem_st_tiles<4>(tmET + 32 * hs + lane_off, Td);
            tmem_wait_st();
        }
        ChainSync cs{bar + kBChain, 0, 0};
        uint32_t par = 0;
        int it = 0;
        for (int c = nchunks - 1; c >= 0; --c, ++it, par ^= 1) {
            const int set = it & 1, valid = min(LC, T - c * LC);
            unsigned char* base = smem + set * PipeSmem::kSet1;
            unsigned char *AR = base + SetSmem::kAR, *BK = base + SetSmem::kBK, *SV = base + SetSmem::kSV, *EY = base + SetSmem::kEY;
            unsigned char *S0 = base + SetSmem::kS0, *Pm = base + SetSmem::kP;
            unsigned char* N1b = base + SetSmem::kN1;
            const float* Lam = reinterpret_cast<const float*>(base + SetSmem::kLam);
            const float* We = reinterpret_cast<const float*>(base + SetSmem::kWe);
            const uint32_t arA = smem_u32(AR), bkA = smem_u32(BK), svA = smem_u32(SV), eyA = smem_u32(EY), s0A = smem_u32(S0);
            const uint32_t uakA = smem_u32(base + SetSmem::kUak), ubrA = smem_u32(base + SetSmem::kUbr), ukrA = smem_u32(base + SetSmem::kUkr);
            const uint32_t d0A = smem_u32(base + SetSmem::kD0), n1A = smem_u32(base + SetSmem::kN1), pA = smem_u32(Pm);
            PIPE_MARK(6);
            if (!mbar_wait(bar + kFull + set, (it >> 1) & 1)) fail = 40;   // the front group has filled this set
            PIPE_MARK(0);
            if (fail) atomicMax(const_cast<int*>(abort_word), fail);
            if (gtid == 0) gabort[1] = *abort_word;
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (gabort[1]) break;
            {   // Ew = E diag(We)  (ETw = diag(We) ET follows under the first products, which do not read it)
                float Ed[4][4];
                tmem_ld_tiles<4>(Ed, tmE + 32 * hs + lane_off);
                tmem_wait_ld();
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const float2 wc = *reinterpret_cast<const float2*>(We + 32 * hs + nt * 8 + 2 * t);
                    Ed[nt][0] *= wc.x; Ed[nt][1] *= wc.y; Ed[nt][2] *= wc.x; Ed[nt][3] *= wc.y;
                }
                tmem_st_tiles<4>(tmE + 32 * hs + lane_off, Ed);
                tmem_wait_st();
            }
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            PIPE_MARK(1);
            // ---- EV, dV ---------------------------------------------------------------------------------
            if (wg == 0) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   // EV0 = Ew B~^T
                    mma_ts(tmW2, tmE + ks * 8, desc_k(bkA, 0, ks * 8, HALF64), idesc64(32, 0, 0), ks > 0, lead);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   //     + dY U_br^T
                    mma_ss(tmW2, desc_mn(eyA + 32 * 128, ks * 8, HALF64), desc_k(ubrA, 0, ks * 8, HALF32), idesc64(32, 1, 0), 1, lead);
                cs.sync(lead);
                issue_solve_t(tmW1, tmW2, d0A, n1A, lead, cs, [&]() {   // EV = EV0 T^T; meanwhile the parts of dV that do not need EV
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)   // dV = Ew K~^T
                        mma_ts(tmW1 + 32, tmE + ks * 8, desc_k(bkA, 32, ks * 8, HALF64), idesc64(32, 0, 0), ks > 0, lead);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)   //    + dY U_kr^T
                        mma_ss(tmW1 + 32, desc_mn(eyA + 32 * 128, ks * 8, HALF64), desc_k(ukrA, 0, ks * 8, HALF32), idesc64(32, 1, 0), 1, lead);
                });
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   //    + EV U_ak^T
                    mma_ts(tmW1 + 32, tmW1 + ks * 8, desc_k(uakA, 0, ks * 8, HALF32), idesc64(32, 0, 0), 1, lead);
                mma_commit(bar + kBEV, lead);
                if (cs.fail) fail = 41;
            }
            // meanwhile, under the chain: SA of this chunk (left in tensor memory by the front group) -> SV rows 0-31
            // ([t][i]; this warp: tokens 16*hs .. 16*hs+15), and ETw = diag(We) ET; both are read by the products after EV only
            if (!mbar_wait(bar + kFSA + set, (it >> 1) & 1)) fail = 46;
            tc_fence_after();
            {
                float sa[2][4];
                tmem_ld_tiles<2>(sa, (set ? tmF2b : tmF2a) + 32 + 16 * hs + lane_off);
                tmem_wait_ld();
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = row0 + g + ((e & 2) ? 8 : 0), tt = 16 * hs + nt * 8 + 2 * t + (e & 1);
                        *reinterpret_cast<float*>(SV + sw(tt, i, HALF64)) = tf32rf(sa[nt][e]);
                    }
            }
            {
                float Td[4][4];
                tmem_ld_tiles<4>(Td, tmET + 32 * hs + lane_off);
                tmem_wait_ld();
                const float wr0 = We[row0 + g], wr1 = We[row0 + g + 8];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) { Td[nt][0] *= wr0; Td[nt][1] *= wr0; Td[nt][2] *= wr1; Td[nt][3] *= wr1; }
                tmem_st_tiles<4>(tmET + 32 * hs + lane_off, Td);
                tmem_wait_st();
            }
            if (!mbar_wait(bar + kBEV, par)) fail = 42;
            tc_fence_after();
            {   // EV -> EY rows 0-31 ([u][i]); dV -> global.  This warp: tokens 16*hs .. 16*hs+15
                float ev[2][4], dv[2][4];
                tmem_ld_tiles<2>(ev, tmW1 + 16 * hs + lane_off);
                tmem_ld_tiles<2>(dv, tmW1 + 32 + 16 * hs + lane_off);
                tmem_wait_ld();
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = row0 + g + ((e & 2) ? 8 : 0), tt = 16 * hs + nt * 8 + 2 * t + (e & 1);
                        *reinterpret_cast<float*>(EY + sw(tt, i, HALF64)) = tf32rf(ev[nt][e]);
                        *reinterpret_cast<bf16*>(N1b + stage_off(tt, i)) = __float2bfloat16_rn(dv[nt][e]);   // N1 is dead: staged, sent with the others
                    }
            }
            proxy_fence();
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            PIPE_MARK(2);
            // ---- P; with it what needs EV but not P ---------------------------------------------------
            if (wg == 0) {
                const uint32_t idkk = idesc64(64, 0, 0), idmm = idesc64(64, 1, 1);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    mma_ss(tmW2, desc_k(eyA, 0, ks * 8, HALF64), desc_k(svA, 0, ks * 8, HALF64), idkk, ks > 0, lead);
                mma_commit(bar + kBP, lead);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   // [dB'|dK'] = ETw [SA;V]^T
                    mma_ts(tmW1, tmET + ks * 8, desc_k(svA, 0, ks * 8, HALF64), idkk, ks > 0, lead);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   // E += [EV;dY] (stacked over tokens) [A~;R~]
                    mma_ss(tmE, desc_mn(eyA, ks * 8, HALF64), desc_mn(arA, ks * 8, HALF64), idmm, 1, lead);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   // ET += [A~;R~]^T [EV;dY]
                    mma_ss(tmET, desc_mn(arA, ks * 8, HALF64), desc_mn(eyA, ks * 8, HALF64), idmm, 1, lead);
                mma_commit(bar + kBE, lead);
            }
            if (!mbar_wait(bar + kBP, par)) fail = 43;
            tc_fence_after();
            {   // masked P -> shared memory
                float p[4][4];
                tmem_ld_tiles<4>(p, tmW2 + 32 * hs + lane_off);
                tmem_wait_ld();
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = row0 + g + 8 * h, u = row & 31, c0 = nt * 8 + 2 * t;
                        const bool strict = row < 32;
                        const float p0 = (strict ? u > c0 : u >= c0) ? p[nt][2 * h] : 0.f;
                        const float p1 = (strict ? u > c0 + 1 : u >= c0 + 1) ? p[nt][2 * h + 1] : 0.f;
                        *reinterpret_cast<float2*>(Pm + sw(row, 32 * hs + c0, HALF64)) = make_float2(tf32rf(p0), tf32rf(p1));
                    }
            }
            proxy_fence();
            tc_fence_before();
            group_sync(gbar, GNT);
            tc_fence_after();
            if (wg == 0) {
                const uint32_t idmm = idesc64(64, 1, 1), idmk = idesc64(64, 1, 0);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   // [dB'|dK'] += [A~;R~]^T P
                    mma_ss(tmW1, desc_mn(arA, ks * 8, HALF64), desc_mn(pA, ks * 8, HALF64), idmm, 1, lead);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   // [dA'|dR'] = S0^T [EV;dY]^T
                    mma_ss(tmW2, desc_mn(s0A, ks * 8, HALF64), desc_k(eyA, 0, ks * 8, HALF64), idmk, ks > 0, lead);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)   //            + [B~;K~]^T P^T
                    mma_ss(tmW2, desc_mn(bkA, ks * 8, HALF64), desc_k(pA, 0, ks * 8, HALF64), idmk, 1, lead);
                mma_commit(bar + kBG, lead);
            }
            PIPE_MARK(3);
            // meanwhile the anchor: A0[j] = sum_i ET_new[j][i] S0[i][j]; this warp: value columns 32*hs .. 32*hs+31
            if (!mbar_wait(bar + kBE, par)) fail = 44;
            tc_fence_after();
            {
                float Td[4][4];
                tmem_ld_tiles<4>(Td, tmET + 32 * hs + lane_off);
                tmem_wait_ld();
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int i = 32 * hs + nt * 8 + 2 * t + e;
                        acc0 = fmaf(Td[nt][e], *reinterpret_cast<const float*>(S0 + sw(i, row0 + g, HALF64)), acc0);
                        acc1 = fmaf(Td[nt][2 + e], *reinterpret_cast<const float*>(S0 + sw(i, row0 + g + 8, HALF64)), acc1);
                    }
                acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1); acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
                acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1); acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
                if (t == 0) { A0p[hs * 64 + row0 + g] = acc0; A0p[hs * 64 + row0 + g + 8] = acc1; }
            }
            if (!mbar_wait(bar + kBG, par)) fail = 45;
            tc_fence_after();
            PIPE_MARK(4);
            // ---- epilogue: this warp has key rows row0+g / +8 and tokens 16*hs .. 16*hs+15 ------------------
            bf16* stg[5];
#pragma unroll
            for (int o = 0; o < 5; ++o) stg[o] = reinterpret_cast<bf16*>((o < 3 ? SV : Pm) + (o < 3 ? o : o - 3) * (32 * 72 * 2));
            float gl[2][2][2], fw[2][2][2];
            {
                float gB[2][4], gK[2][4], gA[2][4], gR[2][4];
                tmem_ld_tiles<2>(gB, tmW1 + 16 * hs + lane_off);
                tmem_ld_tiles<2>(gK, tmW1 + 32 + 16 * hs + lane_off);
                tmem_ld_tiles<2>(gA, tmW2 + 16 * hs + lane_off);
                tmem_ld_tiles<2>(gR, tmW2 + 32 + 16 * hs + lane_off);
                tmem_wait_ld();
                float run[2] = {0.f, 0.f};
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    float ct[2][2];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int j = row0 + g + 8 * h, tt = 16 * hs + nt * 8 + 2 * t + e, x = 2 * h + e;
                            const float at = tf32_seen(AR + sw(tt, j, HALF64)), rt = tf32_seen(AR + sw(32 + tt, j, HALF64));
                            const float bt = tf32_seen(BK + sw(tt, j, HALF64)), kt = tf32_seen(BK + sw(32 + tt, j, HALF64));
                            const float ada = at * gA[nt][x];
                            ct[h][e] = rt * gR[nt][x] + ada - bt * gB[nt][x] - kt * gK[nt][x];
                            gl[h][nt][e] = ada;
                            const float lam = Lam[tt * LAMP + j], lamp = tt > 0 ? Lam[(tt - 1) * LAMP + j] : 0.f;
                            const float wt = fex2(lam), iw = fex2(-lam), wp = fex2(lamp);
                            const float sg = (lam - lamp) * (1.f / kWScale2);
                            fw[h][nt][e] = kWScale * sg * (1.f - sg);
                            stg[0][tt * 72 + j] = __float2bfloat16_rn(gR[nt][x] * wt);
                            stg[1][tt * 72 + j] = __float2bfloat16_rn(gA[nt][x] * wp);
                            stg[2][tt * 72 + j] = __float2bfloat16_rn(gK[nt][x] * iw);
                            stg[3][tt * 72 + j] = __float2bfloat16_rn(gB[nt][x] * iw);
                        }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float pair = ct[h][0] + ct[h][1];
                        float inc = pair;
                        float nb = __shfl_up_sync(0xffffffffu, inc, 1, 4);
                        if (t >= 1) inc += nb;
                        nb = __shfl_up_sync(0xffffffffu, inc, 2, 4);
                        if (t >= 2) inc += nb;
                        const float tot = __shfl_sync(0xffffffffu, inc, 3, 4);
                        const float p0 = run[h] + inc - pair;
                        gl[h][nt][1] += p0 + ct[h][0];
                        gl[h][nt][0] += p0;
                        run[h] += tot;
                    }
                }
                if (hs == 0 && t == 0) { Carry[row0 + g] = run[0]; Carry[row0 + g + 8] = run[1]; }
            }
            tc_fence_before();
            group_sync(gbar, GNT);
            // every product that reads EY or S0 of this set has completed and every thread has taken its anchor from S0:
            // the tiles of the chunk that uses the set next may come
            if (staged && c >= 2) request(set, c - 2);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int j = row0 + g + 8 * h;
                const float a0 = A0p[j] + A0p[64 + j] - (hs ? Carry[j] : 0.f);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int tt = 16 * hs + nt * 8 + 2 * t + e;
                        stg[4][tt * 72 + j] = __float2bfloat16_rn((a0 - gl[h][nt][e]) * fw[h][nt][e]);
                    }
            }
            PIPE_MARK(5);
            group_sync(gbar, GNT);   // all five staged tensors are complete: the front group stores them and refills the set
            if (gtid == 0) mbar_arrive(bar + kEmpty + set);   // the front group may refill this set
        }
        if (fail) atomicMax(const_cast<int*>(abort_word), fail);
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const int ab = *abort_word;
    if (ab && tid == 0) {   // leaving early: tiles that were asked for and not taken must have landed before the block may end
        for (int set = 0; set < 2; ++set)
            for (int k = raw_got[set]; k < raw_req[set]; ++k) mbar_wait(bar + kRaw + set, k & 1);
    }
    if (ab && tid == 0) {   // a wait ran out: record it and poison this unit's outputs so that they cannot pass as results
        atomicMax(&g_l32_bwdp_error, ab);
        dr_[tok0] = __ushort_as_bfloat16((unsigned short)0x7fc0);
    }
    if (!ab && grp == 1 && ds0_ != nullptr) {
        float Ed[4][4];
        tmem_ld_tiles<4>(Ed, tmE + 32 * hs + lane_off);
        tmem_wait_ld();
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            *reinterpret_cast<float2*>(ds0_ + sbase + (row0 + g) * 64 + 32 * hs + nt * 8 + 2 * t) = make_float2(Ed[nt][0], Ed[nt][1]);
            *reinterpret_cast<float2*>(ds0_ + sbase + (row0 + g + 8) * 64 + 32 * hs + nt * 8 + 2 * t) = make_float2(Ed[nt][2], Ed[nt][3]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tm0) : "memory");
}

WKV7_PHASE_READER(rwkvb200_phase_clocks_l32_bwdp)

}  // namespace v7p

int wkv7_l32_backward_pipelined(int B, int T, int H, const void* r, const void* w, const void* k, const void* v, const void* a,
                                const void* b, const void* dy, const float* dsT, const float* s, float* ds0, void* dr, void* dw,
                                void* dk, void* dv, void* da, void* db, cudaStream_t st) {
    using namespace v7p;
    cudaError_t e = cudaFuncSetAttribute(wkv7p_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PipeSmem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_backward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    TileMaps<7> maps;
    const void* in[7] = {r, w, k, v, a, b, dy};
    make_tile_maps<7>(maps, in, B, T, H);
    dim3 grid(H, B);
    wkv7p_backward_kernel<<<grid, PNT, PipeSmem::kBytes, st>>>(T, H, (const bf16*)r, (const bf16*)w, (const bf16*)k,
                                                               (const bf16*)v, (const bf16*)a, (const bf16*)b, (const bf16*)dy,
                                                               dsT, s, ds0, (bf16*)dr, (bf16*)dw, (bf16*)dk, (bf16*)dv,
                                                               (bf16*)da, (bf16*)db, maps);
    return check_launch("wkv7_backward(tcgen05, 32-token chunks, two stages)");
}

int wkv7_l32_bwdp_error(int clear) {
    int h = 0;
    if (clear) return cudaMemcpyToSymbol(v7p::g_l32_bwdp_error, &h, sizeof(int)) == cudaSuccess ? 0 : -1;
    if (cudaMemcpyFromSymbol(&h, v7p::g_l32_bwdp_error, sizeof(int)) != cudaSuccess) return -1;
    return h;
}

}  // namespace rwkvb200
