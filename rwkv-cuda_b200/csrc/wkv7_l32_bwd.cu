// RWKV-7 backward, head size 64, bf16 activations: chunks of 32 tokens, every product on tcgen05.
//
// Walks the chunks in reverse.  Carried across chunks, in tensor memory, are E = dL/dS (lanes = value i,
// columns = key j) and its transpose ET.  Per chunk, with the scaled operands and matrices of
// wkv7_l32.cuh, S0 the saved state at the start of the chunk, Ew = E diag(We):
//   forward part again:   SA = (S0 A~^T + V U_ak) T
//   EV  = (Ew B~^T + dY U_br^T) T^T                            (64 x 32; column t is E_t b_t)
//   dV  =  Ew K~^T + EV U_ak^T + dY U_kr^T
//   P   = [EV;dY]^T [SA;V]   masked: rows from EV keep u > t, rows from dY keep u >= t      (64 x 64)
//   [dB'|dK'] = ETw [SA;V]^T + [A~;R~]^T P          db_t = dB'[:,t] / W_t      dk_t = dK'[:,t] / W_t
//   [dA'|dR'] = S0^T [EV;dY]^T + [B~;K~]^T P^T      da_t = dA'[:,t] W_{t-1}    dr_t = dR'[:,t] W_t
//   E  <- Ew + [EV;dY]^T-stacked [A~;R~]   (and the same for ET, transposed)
// The decay gradient needs no second pass over state pairs: with c_t = r~ dR' + a~ dA' - b~ dB' - k~ dK'
// (per key channel, the scaled vectors exactly as the tensor core saw them, so that the terms that
// cancel between tokens cancel exactly) and A0[j] = sum_i E_new[i,j] S0[i,j],
//   dL/dlog d_t = A0 - sum_{tau<t} c_tau - a~_t dA'_t
// anchored afresh at every chunk so rounding does not accumulate along the sequence.
//
// One CTA of 8 warps per (batch, head), two CTAs per SM.  Warp w works on quarter w%4 of tensor memory
// (16 rows) and, where a region is split, on token half w/4.  Shared memory: six [64][64] operand
// arrays (each read K-major and MN-major as needed), P reusing the space of the U matrices.
// Tensor memory (256 columns): E | ET | W1 | W2, the two work regions reused along the chunk.
#include "wkv7_l32.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7x {

constexpr int BNT = 256;   // threads
constexpr int BTPW = 4;    // tokens per warp in operand preparation

__device__ int g_l32_bwd_error = 0;

struct BwdSmemX {
    static constexpr int kAR = 0;
    static constexpr int kBK = kAR + ARR64;
    static constexpr int kSV = kBK + ARR64;              // rows 0-31 SA_t, rows 32-63 v_t   (columns = value i)
    static constexpr int kEY = kSV + ARR64;              // rows 0-31 EV_u, rows 32-63 dy_u  (columns = value i)
    static constexpr int kS0 = kEY + ARR64;              // [i][j]
    static constexpr int kUak = kS0 + ARR64;             // Uak Ubr Ukr D0: 4 x [32][32]; later P [64][64]
    static constexpr int kUbr = kUak + HALF32;
    static constexpr int kUkr = kUbr + HALF32;
    static constexpr int kD0 = kUkr + HALF32;
    static constexpr int kP = kUak;
    static constexpr int kN1 = kD0 + HALF32;             // [32][32]
    static constexpr int kLam = kN1 + HALF32;            // plain [32][LAMP]: cumulative log2 decays
    static constexpr int kWe = kLam + 32 * LAMP * 4;     // [64]
    static constexpr int kA0 = kWe + 256;                // [2][64] partial anchors
    static constexpr int kCarry = kA0 + 512;             // [64] sum of c over the first 16 tokens
    static constexpr int kBar = kCarry + 256;            // 8 mbarriers + tmem slot
    static constexpr int kBytes = kBar + 128 + 1024;     // + slack to start on a 1024-byte boundary
    // the next chunk's seven input tiles ([32 tokens][64 channels] bf16, 4 KB each) as the copy engine delivers
    // them: in EY and the first 12 KB of S0, which are dead from the last products of a chunk to the preparation of the next
    static constexpr int kRaw = kEY;
    // inside the EV rows of EY (two pieces of 4096 bytes), free until EV is written: the exchange buffer
    // and the two diagonal blocks of U_ab, plain fp32 [2][16][BPITCH]
    static constexpr int kHs = kEY;                      // [8][64]
    static constexpr int kUab = kEY + HALF64;
};
constexpr int BPITCH = 20;
static_assert(2 * 16 * BPITCH * 4 <= HALF32 && 8 * 64 * 4 <= HALF32, "scratch fits in the EV rows");
static_assert(BwdSmemX::kBytes <= 115712, "two CTAs per SM");

// one warp's 16 rows x 32 columns (tiles u[0..3]) of U -> masked matrices; hs = 0: columns a~_t, hs = 1: columns r~_t
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

__device__ __forceinline__ float tf32_seen(const unsigned char* p) {   // operand word -> the value the tensor core used
    return __uint_as_float(*reinterpret_cast<const uint32_t*>(p) & 0xffffe000u);
}

__global__ void __launch_bounds__(BNT, 2)
wkv7x_backward_kernel(int T, int H, const bf16* __restrict__ r_, const bf16* __restrict__ w_,
                      const bf16* __restrict__ k_, const bf16* __restrict__ v_, const bf16* __restrict__ a_,
                      const bf16* __restrict__ b_, const bf16* __restrict__ dy_, const float* __restrict__ dsT_,
                      const float* __restrict__ ck_, float* __restrict__ ds0_, bf16* __restrict__ dr_,
                      bf16* __restrict__ dw_, bf16* __restrict__ dk_, bf16* __restrict__ dv_, bf16* __restrict__ da_,
                      bf16* __restrict__ db_, const __grid_constant__ TileMaps<7> maps) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // the swizzle acts on address bits
    unsigned char *AR = smem + BwdSmemX::kAR, *BK = smem + BwdSmemX::kBK, *SV = smem + BwdSmemX::kSV, *EY = smem + BwdSmemX::kEY;
    unsigned char *S0 = smem + BwdSmemX::kS0, *Uak = smem + BwdSmemX::kUak, *Ubr = smem + BwdSmemX::kUbr, *Ukr = smem + BwdSmemX::kUkr;
    unsigned char *D0 = smem + BwdSmemX::kD0, *N1 = smem + BwdSmemX::kN1, *Pm = smem + BwdSmemX::kP;
    float* Lam = reinterpret_cast<float*>(smem + BwdSmemX::kLam);
    float* We = reinterpret_cast<float*>(smem + BwdSmemX::kWe);
    float* A0p = reinterpret_cast<float*>(smem + BwdSmemX::kA0);
    float* Carry = reinterpret_cast<float*>(smem + BwdSmemX::kCarry);
    float* Hs = reinterpret_cast<float*>(smem + BwdSmemX::kHs);
    float* Uab = reinterpret_cast<float*>(smem + BwdSmemX::kUab);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + BwdSmemX::kBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 8);
    unsigned char* Raw = smem + BwdSmemX::kRaw;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int quarter = warp & 3, hs = warp >> 2;
    const int row0 = quarter * 16;
    const int C = H * 64;
    const i64 tok0 = (i64)bb * T * C + hh * 64;
    const i64 sbase = (i64)(bb * H + hh) * 64 * 64;
    const int nchunks = (T + LC - 1) / LC;
    const float* ck = ck_ + (i64)(bb * H + hh) * (T / 16) * 64 * 64;   // block [b][h] of the caller's (B,H,T/16,N,N) buffer
    const bf16* src[7] = {r_, w_, k_, v_, a_, b_, dy_};

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) mbar_init(bar + i);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < HALF32 / 4; i += BNT) reinterpret_cast<float*>(N1)[i] = 0.f;   // only its upper right block is ever written
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmE = __shfl_sync(0xffffffffu, tmem_slot[0], 0), tmET = tmE + 64, tmW1 = tmE + 128, tmW2 = tmE + 192;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t lead = elect_one();
    const uint32_t arA = smem_u32(AR), bkA = smem_u32(BK), svA = smem_u32(SV), eyA = smem_u32(EY), s0A = smem_u32(S0);
    const uint32_t uakA = smem_u32(Uak), ubrA = smem_u32(Ubr), ukrA = smem_u32(Ukr), d0A = smem_u32(D0), n1A = smem_u32(N1), pA = smem_u32(Pm);

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

    auto fetch_state = [&](int c) {   // chunk-start state -> S0 (swizzled), 16-byte pieces
        const float* s0g = ck + (i64)c * 64 * 64;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            const int idx = q4 * BNT + tid, i = idx >> 4, col = (idx & 15) * 4;
            cp_async16(S0 + sw(i, col, HALF64), s0g + i * 64 + col);
        }
        cp_async_commit();
    };

    RawChunk<7, BTPW> raw;
    // With tensor maps the inputs come by the copy engine: one thread asks for the seven tiles of a chunk (counted in
    // bytes on mbarrier 7) when the arrays that receive them are dead, and at the top of that chunk every thread takes
    // its words out of them; without maps every thread loads its words itself, one chunk ahead, into registers.
    const bool staged = maps.valid != 0;
    bool pending = false;   // a request whose tiles have not been taken yet
    // (called by every thread: lane 0 of warp x asks for tile x, an issue costs a thread about 55 cycles; warp 0
    // announces the bytes, which may happen before or after the other warps' copies complete)
    auto request = [&](int c) {
        if (lane != 0) return;
        if (warp == 0) mbar_expect_bytes(bar + 7, 7 * 4096);
        if (warp < 7) tma_tile_load(Raw + warp * 4096, &maps.m[warp], hh * 64, bb * T + c * LC, bar + 7);
    };
    // the chunk after next into L2: lane 1 of warp x asks for tile x, warp 7 for the chunk-start state
    auto ask_l2 = [&](int c) {
        if (lane != 1 || !maps.valid) return;
        if (warp < 7) l2_prefetch_tile(&maps.m[warp], hh * 64, bb * T + c * LC);
        else {
            const float* sp = ck + (i64)c * 64 * 64;
            if ((reinterpret_cast<uintptr_t>(sp) & 15) == 0) l2_prefetch(sp, 64 * 64 * 4);
        }
    };
    auto take = [&](int c) {
        const int t0 = c * LC + BTPW * warp;
#pragma unroll
        for (int x = 0; x < 7; ++x)
#pragma unroll
            for (int q = 0; q < BTPW; ++q)
                raw.x[x][q] = (t0 + q < T) ? *reinterpret_cast<const uint32_t*>(Raw + x * 4096 + (BTPW * warp + q) * 128 + lane * 4) : 0u;
    };
    if (staged) { request(nchunks - 1); pending = true; }
    else fetch_chunk<7, BTPW>(raw, src, tok0, C, nchunks - 1, T, warp, lane);
    if (nchunks > 1) ask_l2(nchunks - 2);
    int fail = 0;
    uint32_t par = 0;
    ChainSync cs{bar + 6, 0, 0};   // used by warp 0 only

    WKV7_PHASE_BEGIN();
    for (int c = nchunks - 1; c >= 0; --c, par ^= 1) {
        const int valid = min(LC, T - c * LC);
        tc_fence_before();
        if (__syncthreads_or(fail)) break;
        tc_fence_after();
        WKV7_PHASE(0);   // top barrier
        if (staged) {
            if (!mbar_wait(bar + 7, par)) fail = 9;
            take(c);
            pending = false;
            __syncthreads();   // the tiles lie where the state and the scratch of the preparation go next
        }
        fetch_state(c);
        // the zero blocks of D0 (its space was used by P), and N1 (it held the staged dv; only its upper right block is
        // written below, the rest has to read as zero)
        {
            const int s = tid >> 4, cc = tid & 15;   // 16 x 16
            *reinterpret_cast<float*>(D0 + sw32(s, 16 + cc)) = 0.f;
            *reinterpret_cast<float*>(D0 + sw32(16 + s, cc)) = 0.f;
            reinterpret_cast<float4*>(N1)[tid] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // ---- 1. operands ---------------------------------------------------------------------------
        prepare_operands<7, BTPW, 8>(raw, valid, AR, BK, SV + 32 * 128, HALF64, EY + 32 * 128, HALF64, We, Hs, Lam, warp, lane);
        WKV7_PHASE(1);   // operand preparation
        cp_async_wait<0>();   // the chunk-start state
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        WKV7_PHASE(2);   // barrier
        // ---- 2. U ------------------------------------------------------------------------------------
        if (warp == 0) {
            issue_u(tmW1, arA, bkA, lead);
            mma_commit(bar, lead);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // X_a = S0 A~^T, needed after the inverse only
                mma_ss(tmW2, desc_k(s0A, 0, ks * 8, HALF64), desc_k(arA, 0, ks * 8, HALF64), idesc64(32, 0, 0), ks > 0, lead);
        }
        if (!mbar_wait(bar, par)) fail = 1;
        tc_fence_after();
        WKV7_PHASE(3);   // U on the tensor core
        // ---- 3. masked U, inverses of the diagonal blocks -----------------------------------------------
        {
            float u[4][4];
            tmem_ld_tiles<4>(u, tmW1 + 32 * hs + lane_off);
            tmem_wait_ld();
            scatter_u_half(u, quarter, hs, lane, Uab, N1, Uak, Ubr, Ukr);
        }
        tc_fence_before();
        __syncthreads();
        if (warp < 2) tri_inverse16<BPITCH>(Uab + warp * 16 * BPITCH, D0, 16 * warp, lane);
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        WKV7_PHASE(4);   // masked U, inverse
        // ---- 4. the forward part again: SA ----------------------------------------------------------------
        if (warp == 0) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)   // Z = X_a + V U_ak
                mma_ss(tmW2, desc_mn(svA + 32 * 128, ks * 8, HALF64), desc_mn(uakA, ks * 8, HALF32), idesc64(32, 1, 1), 1, lead);
            cs.sync(lead);
            issue_solve(tmW2 + 32, tmW2, d0A, n1A, lead, cs, []() {});   // SA = Z T
            mma_commit(bar + 1, lead);
        }
        // meanwhile: Ew = E diag(We), ETw = diag(We) ET
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
        if (c > 0 && !staged) fetch_chunk<7, BTPW>(raw, src, tok0, C, c - 1, T, warp, lane);   // under the chain
        if (c > 1) ask_l2(c - 2);
        WKV7_PHASE(5);   // issue of the forward part, decay scaling of E, request of the next chunk
        if (!mbar_wait(bar + 1, par)) fail = 2;
        tc_fence_after();
        WKV7_PHASE(6);   // wait for SA
        {   // SA -> SV rows 0-31 ([t][i]); this warp: tokens 16*hs .. 16*hs+15
            float sa[2][4];
            tmem_ld_tiles<2>(sa, tmW2 + 32 + 16 * hs + lane_off);
            tmem_wait_ld();
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = row0 + g + ((e & 2) ? 8 : 0), tt = 16 * hs + nt * 8 + 2 * t + (e & 1);
                    *reinterpret_cast<float*>(SV + sw(tt, i, HALF64)) = tf32rf(sa[nt][e]);
                }
        }
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        WKV7_PHASE(7);   // SA to shared memory
        // ---- 5. EV, dV ------------------------------------------------------------------------------------
        if (warp == 0) {
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
            mma_commit(bar + 2, lead);
            if (cs.fail) fail = 6;
        }
        if (!mbar_wait(bar + 2, par)) fail = 3;
        tc_fence_after();
        WKV7_PHASE(8);   // EV, dV on the tensor core
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
                    *reinterpret_cast<bf16*>(N1 + stage_off(tt, i)) = __float2bfloat16_rn(dv[nt][e]);   // N1 is dead: staged, sent with the others
                }
        }
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        WKV7_PHASE(9);   // EV to shared memory, dv out
        // ---- 6. P; with it what needs EV but not P: the E^T part of [dB'|dK'] and the state gradient ------
        if (warp == 0) {
            const uint32_t idkk = idesc64(64, 0, 0), idmm = idesc64(64, 1, 1);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                mma_ss(tmW2, desc_k(eyA, 0, ks * 8, HALF64), desc_k(svA, 0, ks * 8, HALF64), idkk, ks > 0, lead);
            mma_commit(bar + 3, lead);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // [dB'|dK'] = ETw [SA;V]^T
                mma_ts(tmW1, tmET + ks * 8, desc_k(svA, 0, ks * 8, HALF64), idkk, ks > 0, lead);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // E += [EV;dY] (stacked over tokens) [A~;R~]
                mma_ss(tmE, desc_mn(eyA, ks * 8, HALF64), desc_mn(arA, ks * 8, HALF64), idmm, 1, lead);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)   // ET += [A~;R~]^T [EV;dY]
                mma_ss(tmET, desc_mn(arA, ks * 8, HALF64), desc_mn(eyA, ks * 8, HALF64), idmm, 1, lead);
            mma_commit(bar + 4, lead);
        }
        if (!mbar_wait(bar + 3, par)) fail = 4;
        tc_fence_after();
        WKV7_PHASE(10);  // P on the tensor core
        {   // masked P -> shared memory; rows u (0-31 from EV: u > t, 32-63 from dY: u >= t), columns t (SA | V)
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
        __syncthreads();
        tc_fence_after();
        WKV7_PHASE(11);  // P to shared memory
        // ---- 7. the parts of the gradients of the scaled vectors that need P --------------------------
        if (warp == 0) {
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
            mma_commit(bar + 5, lead);
        }
        // meanwhile the anchor: A0[j] = sum_i ET_new[j][i] S0[i][j]; this warp: value columns 32*hs .. 32*hs+31
        if (!mbar_wait(bar + 4, par)) fail = 5;
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
        if (!mbar_wait(bar + 5, par)) fail = 7;
        tc_fence_after();
        WKV7_PHASE(12);  // final products on the tensor core, anchor
        // ---- 8. epilogue: this warp has key rows row0+g / +8 and tokens 16*hs .. 16*hs+15 ---------------
        // Outputs go through staging rows in shared memory that is dead by now ([32 tokens][72] bf16 each:
        // dr, da, dk in the SA/V array, db, dw in the P array) and leave as 16-byte pieces.
        bf16* stg[5];
#pragma unroll
        for (int o = 0; o < 5; ++o) stg[o] = reinterpret_cast<bf16*>((o < 3 ? SV : Pm) + (o < 3 ? o : o - 3) * (32 * 72 * 2));
        float gl[2][2][2];      // [row][tile][e]: sum of c over the earlier tokens of this half + a~ dA'
        float fw[2][2][2];      // d log-decay / d raw decay input
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
                // exclusive prefix over the tokens of this tile (token = 2*t + e across the four lanes of a quad)
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
        __syncthreads();
        // every product that reads EY or S0 has completed and every thread has taken its anchor from S0
        if (staged && c > 0) { request(c - 1); pending = true; }
        WKV7_PHASE(13);  // epilogue part 1
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
        {   // dr, da, dk, db out: thread = (token, 16-byte piece)
            const int tt = tid >> 3, piece = tid & 7;
            if (tt < valid) {
                const i64 o = tok0 + (i64)(c * LC + tt) * C + piece * 8;
                *reinterpret_cast<uint4*>(dr_ + o) = *reinterpret_cast<const uint4*>(stg[0] + tt * 72 + piece * 8);
                *reinterpret_cast<uint4*>(da_ + o) = *reinterpret_cast<const uint4*>(stg[1] + tt * 72 + piece * 8);
                *reinterpret_cast<uint4*>(dk_ + o) = *reinterpret_cast<const uint4*>(stg[2] + tt * 72 + piece * 8);
                *reinterpret_cast<uint4*>(db_ + o) = *reinterpret_cast<const uint4*>(stg[3] + tt * 72 + piece * 8);
            }
        }
        stage_flush(N1, dv_, tok0 + (i64)c * LC * C, C, tid, valid);
        __syncthreads();
        {
            const int tt = tid >> 3, piece = tid & 7;
            if (tt < valid)
                *reinterpret_cast<uint4*>(dw_ + tok0 + (i64)(c * LC + tt) * C + piece * 8) = *reinterpret_cast<const uint4*>(stg[4] + tt * 72 + piece * 8);
        }
        WKV7_PHASE(14);  // dw out
    }

    if (pending) mbar_wait(bar + 7, par);   // leaving early: the requested tiles must have landed before the block may end
    if (fail && tid == 0) {   // a wait ran out: record it and poison this unit's outputs so that they cannot pass as results
        atomicMax(&g_l32_bwd_error, fail);
        dr_[tok0] = __ushort_as_bfloat16((unsigned short)0x7fc0);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (!fail && ds0_ != nullptr) {
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
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmE) : "memory");
}

WKV7_PHASE_READER(rwkvb200_phase_clocks_l32_bwd)

}  // namespace v7x

int wkv7_l32_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v, const void* a,
                      const void* b, const void* dy, const float* dsT, const float* s, float* ds0, void* dr, void* dw,
                      void* dk, void* dv, void* da, void* db, cudaStream_t st) {
    using namespace v7x;
    cudaError_t e = cudaFuncSetAttribute(wkv7x_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmemX::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_backward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    TileMaps<7> maps;
    const void* in[7] = {r, w, k, v, a, b, dy};
    make_tile_maps<7>(maps, in, B, T, H);
    dim3 grid(H, B);
    wkv7x_backward_kernel<<<grid, BNT, BwdSmemX::kBytes, st>>>(T, H, (const bf16*)r, (const bf16*)w, (const bf16*)k,
                                                               (const bf16*)v, (const bf16*)a, (const bf16*)b, (const bf16*)dy,
                                                               dsT, s, ds0, (bf16*)dr, (bf16*)dw, (bf16*)dk, (bf16*)dv,
                                                               (bf16*)da, (bf16*)db, maps);
    return check_launch("wkv7_backward(tcgen05, 32-token chunks)");
}

int wkv7_l32_bwd_error_clear() {
    const int z = 0;
    return cudaMemcpyToSymbol(v7x::g_l32_bwd_error, &z, sizeof(int)) == cudaSuccess ? 0 : -1;
}

int wkv7_l32_bwd_error() {
    int h = 0;
    if (cudaMemcpyFromSymbol(&h, v7x::g_l32_bwd_error, sizeof(int)) != cudaSuccess) return -1;
    return h;
}

}  // namespace rwkvb200
