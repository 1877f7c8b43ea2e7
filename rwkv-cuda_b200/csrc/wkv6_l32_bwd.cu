// RWKV-6 / RWKV-5 backward, head size 64, bf16 activations: chunks of 32 tokens, every product on tcgen05
// (the structure of wkv7_l32_bwd.cu without the delta-rule terms).
//
// Walks the chunks in reverse.  Carried across chunks, in tensor memory, are E = dL/dS (lanes = value i,
// columns = key j) and its transpose ET.  Per chunk, with the scaled vectors of wkv6_l32_fwd.cu
// (r~_t = r_t P_{t-1}, k~_s = k_s / P_s, k^_s = u k_s / P_{s-1}), S0 the saved state at the start of the
// chunk, Ew = E diag(We), dY = [gy_t] and V = [v_s] (rows = tokens, columns = value i):
//   A[s,t] = k~_s . r~_t (s < t),  A[t,t] = k^_t . r~_t              ([K~;K^] R~^T, as in the forward)
//   G'     = V dY^T:   G[s,t] = G'[s,t] (s < t),   gamma_t = G'[t,t]
//   dV     = Ew K~^T + dY A^T                                              (64 x 32, column s is dv_s)
//   dK'^T  = ETw V^T + R~^T G^T      dk_t = dK'[t] / P_t     + gamma_t u r_t
//   dR'^T  = S0^T dY^T + K~^T G      dr_t = dR'[t] P_{t-1}   + gamma_t u k_t
//   gu     = sum_t gamma_t r_t k_t
//   E  <- Ew + dY^T-stacked R~   (and the same for ET, transposed)
// Decay gradient, anchored at every chunk: with c_t = r~_t dR'_t - k~_t dK'_t (per key channel, the scaled
// vectors as the tensor core saw them) and A0[j] = sum_i E_new[i,j] S0[i,j]:
//   dL/dlog w_t = A0 - sum_{tau<t} c_tau - r~_t dR'_t,     gw_t = dL/dlog w_t * log w_t
// (log w = -exp(w_raw): its derivative by w_raw is log w itself; wkv6_cuda_v1.cu:203 of the reference).  A static
// decay (RWKV-5) has one gw per channel and batch row: the sum over the tokens.
//
// One CTA of 8 warps per (batch, head), two CTAs per SM.  Tensor memory (256 columns): E | ET | W1 (G', then dV) |
// U (the A product) | W2 (dK'^T | dR'^T).  The chunk-start states come from a pass of the forward kernel that
// saves them every 32 tokens.
#include "wkv7_l32.cuh"
#include "wkv6_chunked.cuh"

namespace rwkvb200 {
namespace v6b {

using namespace v7x;

constexpr int BNT = 256;
constexpr int BTPW = 4;

__device__ int g_v6b_error = 0;

struct Smem {
    static constexpr int kRT = 0;                        // [32][64] r~_t
    static constexpr int kKK = kRT + ARR32;              // [64][64] rows 0-31 k~_s, rows 32-63 k^_s
    static constexpr int kVY = kKK + ARR64;              // [64][64] rows 0-31 v_s, rows 32-63 gy_t (columns = value i)
    static constexpr int kS0 = kVY + ARR64;              // [i][j]
    static constexpr int kAm = kS0 + ARR64;              // [32][32] A[s][t]
    static constexpr int kGm = kAm + HALF32;             // [32][32] G[s][t], strict
    static constexpr int kLam = kGm + HALF32;            // plain [32][LAMP]: log2 P_t
    static constexpr int kWe = kLam + 32 * LAMP * 4;
    static constexpr int kA0 = kWe + 256;                // [2][64]
    static constexpr int kCarry = kA0 + 512;             // [64]
    static constexpr int kGam = kCarry + 256;            // [32]
    static constexpr int kBar = kGam + 128;              // 7 mbarriers + tmem slot
    static constexpr int kRaw = kBar + 128;              // the next chunk's inputs as the copy engine delivers them:
                                                         // r, k, v, gy [32][64] bf16 each, then the decay input (bf16 or fp32)
    static constexpr int kBytes = kRaw + 4 * 4096 + 8192 + 1024;
    static constexpr int kHs = kAm;                      // [8][64] exchange buffer of the preparation (A, G not yet written)
};
static_assert(Smem::kBytes <= 115712 && 8 * 64 * 4 <= 2 * HALF32, "two CTAs per SM");

__device__ __forceinline__ float tf32_seen(const unsigned char* p) {
    return __uint_as_float(*reinterpret_cast<const uint32_t*>(p) & 0xffffe000u);
}
__device__ __forceinline__ void store_state(void* p, int kind, i64 idx, float x) {
    if (kind == 2) reinterpret_cast<float*>(p)[idx] = x;
    else if (kind == 1) reinterpret_cast<bf16*>(p)[idx] = __float2bfloat16_rn(x);
}

// WMODE as in wkv6_l32_fwd.cu: 0 = fp32 log-decay (B,T,C), 1 = bf16 raw input (B,T,C), 2 = fp32 decay value (C),
// 3 = fp32 log-decay (C)
template <int WMODE>
__global__ void __launch_bounds__(BNT, 2)
wkv6b_backward_kernel(int T, int H, const bf16* __restrict__ r_, const bf16* __restrict__ k_, const bf16* __restrict__ v_,
                      const void* __restrict__ w_, const bf16* __restrict__ u_, const bf16* __restrict__ gy_,
                      const float* __restrict__ dsT_, const float* __restrict__ ck_, bf16* __restrict__ gr_,
                      bf16* __restrict__ gk_, bf16* __restrict__ gv_, bf16* __restrict__ gw_, bf16* __restrict__ gu_,
                      void* __restrict__ ds0_, int ds0_kind, float* __restrict__ gw32_, float* __restrict__ gu32_,
                      const __grid_constant__ TileMaps<5> maps) {
    constexpr bool kStatic = WMODE >= 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *RT = smem + Smem::kRT, *KK = smem + Smem::kKK, *VY = smem + Smem::kVY, *S0 = smem + Smem::kS0;
    unsigned char *Am = smem + Smem::kAm, *Gm = smem + Smem::kGm;
    float* Lam = reinterpret_cast<float*>(smem + Smem::kLam);
    float* We = reinterpret_cast<float*>(smem + Smem::kWe);
    float* A0p = reinterpret_cast<float*>(smem + Smem::kA0);
    float* Carry = reinterpret_cast<float*>(smem + Smem::kCarry);
    float* Gam = reinterpret_cast<float*>(smem + Smem::kGam);
    float* Hs = reinterpret_cast<float*>(smem + Smem::kHs);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + Smem::kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 7);
    unsigned char* Raw = smem + Smem::kRaw;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int quarter = warp & 3, hs = warp >> 2;
    const int row0 = quarter * 16;
    const int C = H * 64;
    const i64 tok0 = (i64)bb * T * C + hh * 64;
    const i64 sbase = (i64)(bb * H + hh) * 64 * 64;
    const int nchunks = (T + LC - 1) / LC;
    const float* ck = ck_ + (i64)(bb * H + hh) * nchunks * 64 * 64;
    const bf16* src[4] = {r_, k_, v_, gy_};
    const int j0 = 2 * lane;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 7; ++i) mbar_init(bar + i);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmE = __shfl_sync(0xffffffffu, tmem_slot[0], 0), tmET = tmE + 64, tmW1 = tmE + 128, tmU = tmE + 160, tmW2 = tmE + 192;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t lead = elect_one();
    const uint32_t rtA = smem_u32(RT), kkA = smem_u32(KK), vyA = smem_u32(VY), s0A = smem_u32(S0), amA = smem_u32(Am), gmA = smem_u32(Gm);

    // E, ET <- dsT (or zero); this warp: its 16 rows, columns 32*hs .. 32*hs+31
    {
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

    // the bonus of this thread's two rows in the epilogue, and a static decay of the preparation's two channels
    const float ue[2] = {__bfloat162float(u_[hh * 64 + row0 + g]), __bfloat162float(u_[hh * 64 + row0 + g + 8])};
    const float up0 = __bfloat162float(u_[hh * 64 + j0]), up1 = __bfloat162float(u_[hh * 64 + j0 + 1]);
    float ls0 = 0.f, ls1 = 0.f;
    if (WMODE == 2) {
        ls0 = __log2f(reinterpret_cast<const float*>(w_)[hh * 64 + j0]);
        ls1 = __log2f(reinterpret_cast<const float*>(w_)[hh * 64 + j0 + 1]);
    } else if (WMODE == 3) {
        ls0 = reinterpret_cast<const float*>(w_)[hh * 64 + j0] * 1.4426950408889634f;
        ls1 = reinterpret_cast<const float*>(w_)[hh * 64 + j0 + 1] * 1.4426950408889634f;
    }

    RawChunk<4, BTPW> raw;
    // the decay input of this thread's tokens (two channels) as loaded: decoded where it is used, one chunk later, so
    // that nothing waits for the load where it is issued
    uint32_t wraw[BTPW];      // WMODE 1: two bf16
    float2 wlog[BTPW];        // WMODE 0: two fp32 log-decays
    bool win[BTPW];
    auto fetch = [&](int c) {
        fetch_chunk<4, BTPW>(raw, src, tok0, C, c, T, warp, lane);
        const int t0 = c * LC + BTPW * warp;
#pragma unroll
        for (int q = 0; q < BTPW; ++q) {
            const bool in = t0 + q < T;
            win[q] = in;
            if (WMODE == 1) {
                wraw[q] = in ? __ldg(reinterpret_cast<const unsigned int*>(reinterpret_cast<const bf16*>(w_) + tok0 + (i64)(t0 + q) * C + j0)) : 0u;
            } else if (WMODE == 0) {
                wlog[q] = make_float2(0.f, 0.f);
                if (in) wlog[q] = __ldg(reinterpret_cast<const float2*>(reinterpret_cast<const float*>(w_) + tok0 + (i64)(t0 + q) * C + j0));
            }
        }
    };
    // The same through the copy engine, when tensor maps could be made: one thread asks for the tiles of chunk c
    // (counted in bytes on mbarrier 6), and at the top of that chunk every thread takes its words out of the staged tiles.
    constexpr int kRawBytes = 4 * 4096 + (WMODE == 1 ? 4096 : WMODE == 0 ? 8192 : 0);
    // (called by every thread: lane 0 of warp x asks for tile x, an issue costs a thread about 55 cycles; warp 0
    // announces the bytes, which may happen before or after the other warps' copies complete)
    auto request = [&](int c) {
        if (lane != 0) return;
        if (warp == 0) mbar_expect_bytes(bar + 6, kRawBytes);
        if (warp < 4 || (warp == 4 && WMODE <= 1)) tma_tile_load(Raw + warp * 4096, &maps.m[warp], hh * 64, bb * T + c * LC, bar + 6);
    };
    auto take = [&](int c) {
        const int t0 = c * LC + BTPW * warp;
#pragma unroll
        for (int q = 0; q < BTPW; ++q) {
            const bool in = t0 + q < T;
            const int row = BTPW * warp + q;
            win[q] = in;
#pragma unroll
            for (int x = 0; x < 4; ++x) raw.x[x][q] = in ? *reinterpret_cast<const uint32_t*>(Raw + x * 4096 + row * 128 + lane * 4) : 0u;
            if (WMODE == 1) wraw[q] = in ? *reinterpret_cast<const uint32_t*>(Raw + 4 * 4096 + row * 128 + lane * 4) : 0u;
            if (WMODE == 0) wlog[q] = in ? *reinterpret_cast<const float2*>(Raw + 4 * 4096 + row * 256 + lane * 8) : make_float2(0.f, 0.f);
        }
    };
    const bool staged = maps.valid != 0;
    bool pending = false;   // a request whose tiles have not been taken yet
    // log2 decay of token q of the fetched chunk, channels j0 and j0 + 1
    auto decay_log2 = [&](int q, float& l0, float& l1) {
        if (WMODE == 1) {
            const float2 w2 = bf16x2_to_f2(wraw[q]);
            l0 = win[q] ? -fexp(w2.x) * 1.4426950408889634f : 0.f;
            l1 = win[q] ? -fexp(w2.y) * 1.4426950408889634f : 0.f;
        } else if (WMODE == 0) {
            l0 = wlog[q].x * 1.4426950408889634f;
            l1 = wlog[q].y * 1.4426950408889634f;
        } else {
            l0 = win[q] ? ls0 : 0.f;
            l1 = win[q] ? ls1 : 0.f;
        }
    };
    if (!staged) fetch(nchunks - 1);
    else { request(nchunks - 1); pending = true; }
    // two chunks ahead, into L2: the chunk-start state (the input tiles come by the copy engine one chunk ahead)
    auto ask_l2 = [&](int c) {
        if (tid != 224) return;
        const float* sp = ck + (i64)c * 64 * 64;
        if ((reinterpret_cast<uintptr_t>(sp) & 15) == 0) l2_prefetch(sp, 64 * 64 * 4);
    };
    if (nchunks > 1) ask_l2(nchunks - 2);
    int fail = 0;
    uint32_t par = 0;
    float gu_acc[2] = {0.f, 0.f}, gw_acc[2] = {0.f, 0.f};   // sums over this thread's tokens (gw only for a static decay)

    for (int c = nchunks - 1; c >= 0; --c, par ^= 1) {
        const int valid = min(LC, T - c * LC);
        tc_fence_before();
        if (__syncthreads_or(fail)) break;
        tc_fence_after();
        {   // chunk-start state -> S0 (swizzled), 16-byte pieces
            const float* s0g = ck + (i64)c * 64 * 64;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int idx = q4 * BNT + tid, i = idx >> 4, col = (idx & 15) * 4;
                cp_async16(S0 + sw(i, col, HALF64), s0g + i * 64 + col);
            }
            cp_async_commit();
        }
        // ---- 1. operands: this thread has channels j0, j0+1 of tokens 4*warp .. 4*warp+3 ----------------
        if (staged) {
            if (!mbar_wait(bar + 6, par)) fail = 6;
            take(c);
            pending = false;
        }
        {
            float cs0[BTPW], cs1[BTPW], run0 = 0.f, run1 = 0.f;
#pragma unroll
            for (int q = 0; q < BTPW; ++q) {
                float l0, l1;
                decay_log2(q, l0, l1);
                run0 += l0; run1 += l1; cs0[q] = run0; cs1[q] = run1;
            }
            *reinterpret_cast<float2*>(Hs + warp * 64 + j0) = make_float2(run0, run1);
            __syncthreads();
            if (staged && c > 0) { request(c - 1); pending = true; }   // every thread has taken its words: the stage is free
            float base0 = 0.f, base1 = 0.f, tot0 = 0.f, tot1 = 0.f;
#pragma unroll
            for (int gq = 0; gq < 8; ++gq) {
                const float2 h = *reinterpret_cast<const float2*>(Hs + gq * 64 + j0);
                if (gq < warp) { base0 += h.x; base1 += h.y; }
                tot0 += h.x; tot1 += h.y;
            }
            if (warp == 0) *reinterpret_cast<float2*>(We + j0) = make_float2(fex2(tot0), fex2(tot1));
            float lp0 = base0, lp1 = base1;   // log2 P_{t-1}
#pragma unroll
            for (int q = 0; q < BTPW; ++q) {
                const int tt = BTPW * warp + q;
                const float l0 = fmaxf(base0 + cs0[q], -120.f), l1 = fmaxf(base1 + cs1[q], -120.f);
                const float p0 = fmaxf(lp0, -120.f), p1 = fmaxf(lp1, -120.f);
                const float wp0 = fex2(p0), wp1 = fex2(p1), iw0 = fex2(-l0), iw1 = fex2(-l1), ip0 = fex2(-p0), ip1 = fex2(-p1);
                const float2 r2 = bf16x2_to_f2(raw.x[0][q]), k2 = bf16x2_to_f2(raw.x[1][q]);
                *reinterpret_cast<float2*>(RT + sw(tt, j0, HALF32)) = make_float2(tf32rf(r2.x * wp0), tf32rf(r2.y * wp1));
                *reinterpret_cast<float2*>(KK + sw(tt, j0, HALF64)) = make_float2(tf32rf(k2.x * iw0), tf32rf(k2.y * iw1));
                *reinterpret_cast<float2*>(KK + sw(32 + tt, j0, HALF64)) = make_float2(tf32rf(up0 * k2.x * ip0), tf32rf(up1 * k2.y * ip1));
                *reinterpret_cast<float2*>(VY + sw(tt, j0, HALF64)) = bf16x2_to_f2(raw.x[2][q]);
                *reinterpret_cast<float2*>(VY + sw(32 + tt, j0, HALF64)) = bf16x2_to_f2(raw.x[3][q]);
                *reinterpret_cast<float2*>(Lam + tt * LAMP + j0) = make_float2(l0, l1);
                lp0 = base0 + cs0[q]; lp1 = base1 + cs1[q];
            }
        }
        cp_async_wait<0>();
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        // ---- 2. the token x token products ---------------------------------------------------------------
        if (warp == 0) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // [K~;K^] R~^T
                mma_ss(tmU, desc_k(kkA, 0, ks * 8, HALF64), desc_k(rtA, 0, ks * 8, HALF32), idesc64(32, 0, 0), ks > 0, lead);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // G' = [V;dY] dY^T (its rows 0-31 are V dY^T)
                mma_ss(tmW1, desc_k(vyA, 0, ks * 8, HALF64), desc_k(vyA, 32, ks * 8, HALF64), idesc64(32, 0, 0), ks > 0, lead);
            mma_commit(bar, lead);
        }
        // meanwhile: Ew = E diag(We), ETw = diag(We) ET, and the request of the next chunk
        {
            float Ed[4][4], Td[4][4];
            tmem_ld_tiles<4>(Ed, tmE + 32 * hs + lane_off);
            tmem_ld_tiles<4>(Td, tmET + 32 * hs + lane_off);
            tmem_wait_ld();
            const float wr0 = We[row0 + g], wr1 = We[row0 + g + 8];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float2 wc = *reinterpret_cast<const float2*>(We + 32 * hs + nt * 8 + 2 * t);
                Ed[nt][0] *= wc.x; Ed[nt][1] *= wc.y; Ed[nt][2] *= wc.x; Ed[nt][3] *= wc.y;
                Td[nt][0] *= wr0; Td[nt][1] *= wr0; Td[nt][2] *= wr1; Td[nt][3] *= wr1;
            }
            tmem_st_tiles<4>(tmE + 32 * hs + lane_off, Ed);
            tmem_st_tiles<4>(tmET + 32 * hs + lane_off, Td);
            tmem_wait_st();
        }
        if (c > 0 && !staged) fetch(c - 1);
        if (c > 1) ask_l2(c - 2);
        if (!mbar_wait(bar, par)) fail = 1;
        tc_fence_after();
        // ---- 3. A and G masked into shared memory; this warp: rows of its quarter, columns 16*hs .. 16*hs+15 ---
        {
            float ua[2][4], gg[2][4];
            tmem_ld_tiles<2>(ua, tmU + 16 * hs + lane_off);
            tmem_ld_tiles<2>(gg, tmW1 + 16 * hs + lane_off);
            tmem_wait_ld();
            const int sb = 16 * (quarter & 1) + g;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int s = sb + 8 * h, tc = 16 * hs + nt * 8 + 2 * t + e, x = 2 * h + e;
                        if (quarter < 2) {   // rows k~_s / v_s
                            if (s != tc) *reinterpret_cast<float*>(Am + sw32(s, tc)) = s < tc ? tf32rf(ua[nt][x]) : 0.f;
                            *reinterpret_cast<float*>(Gm + sw32(s, tc)) = s < tc ? tf32rf(gg[nt][x]) : 0.f;
                            if (s == tc) Gam[s] = gg[nt][x];
                        } else {             // rows k^_s: the diagonal of A
                            if (s == tc) *reinterpret_cast<float*>(Am + sw32(s, tc)) = tf32rf(ua[nt][x]);
                        }
                    }
        }
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        // ---- 4. the gradients on the tensor core ------------------------------------------------------------
        if (warp == 0) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // dV = Ew K~^T
                mma_ts(tmW1, tmE + ks * 8, desc_k(kkA, 0, ks * 8, HALF64), idesc64(32, 0, 0), ks > 0, lead);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   //    + dY A^T
                mma_ss(tmW1, desc_mn(vyA + 32 * 128, ks * 8, HALF64), desc_k(amA, 0, ks * 8, HALF32), idesc64(32, 1, 0), 1, lead);
            mma_commit(bar + 1, lead);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // dK'^T = ETw V^T
                mma_ts(tmW2, tmET + ks * 8, desc_k(vyA, 0, ks * 8, HALF64), idesc64(32, 0, 0), ks > 0, lead);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   //       + R~^T G^T
                mma_ss(tmW2, desc_mn(rtA, ks * 8, HALF32), desc_k(gmA, 0, ks * 8, HALF32), idesc64(32, 1, 0), 1, lead);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // dR'^T = S0^T dY^T
                mma_ss(tmW2 + 32, desc_mn(s0A, ks * 8, HALF64), desc_k(vyA, 32, ks * 8, HALF64), idesc64(32, 1, 0), ks > 0, lead);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   //       + K~^T G
                mma_ss(tmW2 + 32, desc_mn(kkA, ks * 8, HALF64), desc_mn(gmA, ks * 8, HALF32), idesc64(32, 1, 1), 1, lead);
            mma_commit(bar + 2, lead);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // E += dY (stacked over tokens) R~
                mma_ss(tmE, desc_mn(vyA + 32 * 128, ks * 8, HALF64), desc_mn(rtA, ks * 8, HALF32), idesc64(64, 1, 1), 1, lead);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // ET += R~^T dY
                mma_ss(tmET, desc_mn(rtA, ks * 8, HALF32), desc_mn(vyA + 32 * 128, ks * 8, HALF64), idesc64(64, 1, 1), 1, lead);
            mma_commit(bar + 3, lead);
        }
        // ---- 5. dv out: this warp's rows i, tokens 16*hs .. 16*hs+15 -----------------------------------------
        if (!mbar_wait(bar + 1, par)) fail = 2;
        tc_fence_after();
        {
            float dv[2][4];
            tmem_ld_tiles<2>(dv, tmW1 + 16 * hs + lane_off);
            tmem_wait_ld();
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = row0 + g + ((e & 2) ? 8 : 0), tt = 16 * hs + nt * 8 + 2 * t + (e & 1);
                    if (tt < valid) gv_[tok0 + (i64)(c * LC + tt) * C + i] = __float2bfloat16_rn(dv[nt][e]);
                }
        }
        // ---- 6. the anchor A0[j] = sum_i ET_new[j][i] S0[i][j]; this warp: value columns 32*hs .. 32*hs+31 -----
        if (!mbar_wait(bar + 3, par)) fail = 4;
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
        if (!mbar_wait(bar + 2, par)) fail = 3;
        tc_fence_after();
        // ---- 7. epilogue: this warp has key rows row0+g / +8 and tokens 16*hs .. 16*hs+15 ---------------------
        // staging rows ([32 tokens][72] bf16 each: gr, gk, gw) in the V / gy array, dead by now
        bf16* stg[3];
#pragma unroll
        for (int o = 0; o < 3; ++o) stg[o] = reinterpret_cast<bf16*>(VY + o * (32 * 72 * 2));
        float gl[2][2][2], lw[2][2][2];
        {
            float gK[2][4], gR[2][4];
            tmem_ld_tiles<2>(gK, tmW2 + 16 * hs + lane_off);
            tmem_ld_tiles<2>(gR, tmW2 + 32 + 16 * hs + lane_off);
            tmem_wait_ld();
            // the operand words are read before the staging rows overwrite anything: RT, KK, Lam are other arrays
            float run[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                float ct[2][2];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = row0 + g + 8 * h, tt = 16 * hs + nt * 8 + 2 * t + e, x = 2 * h + e;
                        const float rt = tf32_seen(RT + sw(tt, j, HALF32)), kt = tf32_seen(KK + sw(tt, j, HALF64));
                        const float lam = Lam[tt * LAMP + j], lamp = tt > 0 ? Lam[(tt - 1) * LAMP + j] : 0.f;
                        const float wp = fex2(lamp), iw = fex2(-lam);
                        const float drs = gR[nt][x] * wp, dks = gK[nt][x] * iw;
                        const float rr = rt * fex2(-lamp), kr = kt * fex2(lam);   // r_t, k_t
                        const float gam_u = Gam[tt] * ue[h];
                        const float rdr = rt * gR[nt][x];
                        ct[h][e] = rdr - kt * gK[nt][x];
                        gl[h][nt][e] = rdr;
                        lw[h][nt][e] = (lam - lamp) * 0.6931471805599453f;   // log w_t
                        gu_acc[h] = fmaf(Gam[tt], rr * kr, gu_acc[h]);
                        stg[0][tt * 72 + j] = __float2bfloat16_rn(fmaf(gam_u, kr, drs));
                        stg[1][tt * 72 + j] = __float2bfloat16_rn(fmaf(gam_u, rr, dks));
                    }
#pragma unroll
                for (int h = 0; h < 2; ++h) {   // exclusive prefix over the tokens of this tile (token = 2*t + e over a quad)
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
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int j = row0 + g + 8 * h;
            const float a0 = A0p[j] + A0p[64 + j] - (hs ? Carry[j] : 0.f);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int tt = 16 * hs + nt * 8 + 2 * t + e;
                    const float gw = (a0 - gl[h][nt][e]) * lw[h][nt][e];
                    if (kStatic) gw_acc[h] += gw;
                    else stg[2][tt * 72 + j] = __float2bfloat16_rn(gw);
                }
        }
        {   // gr, gk out: thread = (token, 16-byte piece)
            const int tt = tid >> 3, piece = tid & 7;
            if (tt < valid) {
                const i64 o = tok0 + (i64)(c * LC + tt) * C + piece * 8;
                *reinterpret_cast<uint4*>(gr_ + o) = *reinterpret_cast<const uint4*>(stg[0] + tt * 72 + piece * 8);
                *reinterpret_cast<uint4*>(gk_ + o) = *reinterpret_cast<const uint4*>(stg[1] + tt * 72 + piece * 8);
            }
        }
        if (!kStatic) {
            __syncthreads();
            const int tt = tid >> 3, piece = tid & 7;
            if (tt < valid)
                *reinterpret_cast<uint4*>(gw_ + tok0 + (i64)(c * LC + tt) * C + piece * 8) = *reinterpret_cast<const uint4*>(stg[2] + tt * 72 + piece * 8);
        }
    }

    if (pending) mbar_wait(bar + 6, par);   // leaving early: the requested tiles must have landed before the block may end
    if (fail && tid == 0) {   // a wait ran out: record it and poison this unit's outputs
        atomicMax(&g_v6b_error, fail);
        gr_[tok0] = __ushort_as_bfloat16((unsigned short)0x7fc0);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // gu (and gw of a static decay): sums over the four lanes of a quad and the two token halves
    {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            gu_acc[h] += __shfl_xor_sync(0xffffffffu, gu_acc[h], 1);
            gu_acc[h] += __shfl_xor_sync(0xffffffffu, gu_acc[h], 2);
            gw_acc[h] += __shfl_xor_sync(0xffffffffu, gw_acc[h], 1);
            gw_acc[h] += __shfl_xor_sync(0xffffffffu, gw_acc[h], 2);
        }
        if (hs == 1 && t == 0) {
            A0p[row0 + g] = gu_acc[0]; A0p[row0 + g + 8] = gu_acc[1];
            A0p[64 + row0 + g] = gw_acc[0]; A0p[64 + row0 + g + 8] = gw_acc[1];
        }
        __syncthreads();
        if (hs == 0 && t == 0 && !fail) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int j = row0 + g + 8 * h;
                const float gu = gu_acc[h] + A0p[j], gw = gw_acc[h] + A0p[64 + j];
                gu_[(i64)bb * C + hh * 64 + j] = __float2bfloat16_rn(gu);
                if (gu32_ != nullptr) gu32_[(i64)bb * C + hh * 64 + j] = gu;
                if (kStatic) {
                    gw_[(i64)bb * C + hh * 64 + j] = __float2bfloat16_rn(gw);
                    if (gw32_ != nullptr) gw32_[(i64)bb * C + hh * 64 + j] = gw;
                }
            }
        }
    }
    if (!fail && ds0_kind != 0) {
        float Ed[4][4];
        tmem_ld_tiles<4>(Ed, tmE + 32 * hs + lane_off);
        tmem_wait_ld();
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                store_state(ds0_, ds0_kind, sbase + (row0 + g + ((e & 2) ? 8 : 0)) * 64 + 32 * hs + nt * 8 + 2 * t + (e & 1), Ed[nt][e]);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmE) : "memory");
}

}  // namespace v6b

// Arguments as wkv6_chunked_backward; ck holds the chunk-start states every 32 tokens ((B,H,ceil(T/32),N,N) fp32, written
// by wkv6_l32_forward with its `ck` argument).
int wkv6_l32_backward(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode, const void* u,
                      const void* gy, const float* dsT, const float* ck, void* gr, void* gk, void* gv, void* gw, void* gu,
                      void* ds0, int ds0_kind, cudaStream_t st, float* gw32, float* gu32) {
    using namespace v6b;
    TileMaps<5> maps;
    const void* in[5] = {r, k, v, gy, w_mode <= 1 ? w : r};
    maps.valid = 1;
    for (int x = 0; x < 5 && maps.valid; ++x)
        if (!wkv6_make_tile_map(&maps.m[x], in[x], (unsigned long long)B * T, (unsigned long long)H * 64, x == 4 && w_mode == 0)) maps.valid = 0;
    dim3 grid(H, B);
#define RWKV_GO(M)                                                                                                        \
    do {                                                                                                                  \
        cudaError_t e = cudaFuncSetAttribute(wkv6b_backward_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes); \
        RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv6_backward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));  \
        wkv6b_backward_kernel<M><<<grid, BNT, Smem::kBytes, st>>>(T, H, (const bf16*)r, (const bf16*)k, (const bf16*)v, w,  \
                                                                 (const bf16*)u, (const bf16*)gy, dsT, ck, (bf16*)gr,    \
                                                                 (bf16*)gk, (bf16*)gv, (bf16*)gw, (bf16*)gu, ds0,        \
                                                                 ds0_kind, gw32, gu32, maps);                            \
    } while (0)
    switch (w_mode) {
        case 0: RWKV_GO(0); break;
        case 1: RWKV_GO(1); break;
        case 2: RWKV_GO(2); break;
        default: RWKV_GO(3); break;
    }
#undef RWKV_GO
    return check_launch("wkv6_backward(tcgen05, 32-token chunks)");
}

int wkv6_l32_bwd_error(int clear) {
    int h = 0;
    if (clear) return cudaMemcpyToSymbol(v6b::g_v6b_error, &h, sizeof(int)) == cudaSuccess ? 0 : -1;
    if (cudaMemcpyFromSymbol(&h, v6b::g_v6b_error, sizeof(int)) != cudaSuccess) return -1;
    return h;
}

}  // namespace rwkvb200
