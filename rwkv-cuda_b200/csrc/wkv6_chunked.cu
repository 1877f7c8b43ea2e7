// RWKV-6 forward, head size 64, bf16 activations: chunked tensor-core kernel (mma.sync TF32).
//
// S is [value i][key j]; per token  y_t = S_{t-1} r_t + (r_t.u.k_t) v_t,  S_t = S_{t-1} diag(w_t) + v_t k_t^T
// (wkv6/cuda/wkv6_cuda_v1.cu:24-56).  Within a chunk of L = 16 tokens let P_t = prod_{tau<=t} w_tau
// (per key channel), P_{-1} = 1, We = P_15 and  r~_t = r_t*P_{t-1},  k~_s = k_s/P_s.  Then with S0 the
// state at the start of the chunk, V = [v_t], Y = [y_t] (64 x 16):
//   A[s,t] = k~_s.r~_t (s < t),  A[t,t] = sum_j r_t[j] u[j] k_t[j]
//   Y = S0 R~ + V A          S_end = (S0 + V K~) diag(We)
// i.e. the RWKV-7 chunk (chunk_tf32.cuh) without the a/b terms: no inverse, one 16x16 matrix.
// One CTA of 4 warps per (batch, head); warp w owns state rows 16w..16w+15 as accumulator tiles
// for the whole sequence.
//
// The division by P_s is only safe while a chunk's cumulative decay stays representable: RWKV-6
// has no clamp on w.  The kernel therefore raises a flag when the summed log-decay of any channel
// over a chunk exceeds 80 (P < 1.8e-35); the launcher then runs the general-shape kernel over the
// same problem (it starts by reading the flag, and returns at once when the flag is clear).
#include "chunk_tf32.cuh"
#include "wkv6_chunked.cuh"
#include <atomic>
#include <mutex>

namespace rwkvb200 {
namespace v6c {

using namespace v7c;

constexpr float kMaxChunkLog2Decay = 80.f * 1.4426950408889634f;

struct FSmem {                                                       // floats
    static constexpr int kRawBytes = 2 * 3 * L * N * 2;              // bf16 [2][3][L][N]: r k v
    static constexpr int kRt = kRawBytes / 4;                        // r~      [L][PK], channels permuted
    static constexpr int kKt = kRt + L * PK;                         // k~
    static constexpr int kVf = kKt + L * PK;                         // v
    static constexpr int kRu = kVf + L * PK;                         // r*u
    static constexpr int kKr = kRu + L * PK;                         // k
    static constexpr int kAT = kKr + L * PK;                         // A stored [t][s]
    static constexpr int kWe = kAT + L * PU;
    static constexpr int kHalf = kWe + N;
    static constexpr int kEnd = kHalf + 2 * N;                      // [2][N] half-chunk log-decay sums
    static constexpr int kBytes = kEnd * 4;
};

// The decay input of one (token, channel), fetched one chunk ahead as raw bits and turned into the
// log2 of the decay only where it is used (arithmetic right behind the load would make the warp wait
// for it).  w_mode 0 = fp32 log-decay (B,T,C), 1 = bf16 raw input (B,T,C), log-decay = -exp(w);
// static per channel (RWKV-5): 2 = fp32 decay value (C), 3 = fp32 log-decay (C).
// (volatile asm: the compiler must issue the load here, not sink it to the first use a chunk later)
template <int mode>
__device__ __forceinline__ uint32_t decay_bits(const void* w, i64 tok_idx, int ch_idx) {
    uint32_t x;
    if (mode == 1) {
        unsigned short h;
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(h) : "l"(reinterpret_cast<const unsigned short*>(w) + tok_idx));
        x = (uint32_t)h << 16;
    } else {
        asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(x) : "l"(reinterpret_cast<const uint32_t*>(w) + (mode == 0 ? tok_idx : (i64)ch_idx)));
    }
    return x;
}
template <int mode>
__device__ __forceinline__ float decay_log2(uint32_t bits) {
    const float x = __uint_as_float(bits);
    if (mode == 1) return -fexp(x) * 1.4426950408889634f;
    if (mode == 2) return __log2f(x);
    return x * 1.4426950408889634f;
}

__device__ __forceinline__ float load_s0(const void* p, int kind, i64 idx) {
    if (kind == 2) return reinterpret_cast<const float*>(p)[idx];
    if (kind == 1) return __bfloat162float(reinterpret_cast<const bf16*>(p)[idx]);
    return 0.f;
}

// STATES_ONLY: the pass of the backward that only rebuilds the chunk-start states (no r, no A, no y).
template <int WMODE, bool STATES_ONLY>
__global__ void __launch_bounds__(NT, 4)
wkv6c_forward_kernel(int T, int H, const bf16* __restrict__ r_, const bf16* __restrict__ k_,
                     const bf16* __restrict__ v_, const void* __restrict__ w_, const bf16* __restrict__ u_,
                     const void* __restrict__ s0_, int s0_kind, bf16* __restrict__ y_, float* __restrict__ sT_,
                     float* __restrict__ ck_, int* __restrict__ unsafe_, int flag_div) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* sm = reinterpret_cast<float*>(smem_raw);
    bf16* raw = reinterpret_cast<bf16*>(smem_raw);
    float *Rt = sm + FSmem::kRt, *Kt = sm + FSmem::kKt, *Vf = sm + FSmem::kVf, *Ru = sm + FSmem::kRu, *Kr = sm + FSmem::kKr;
    float *AT = sm + FSmem::kAT, *We = sm + FSmem::kWe, *Hs = sm + FSmem::kHalf;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = warp * 16;
    const int C = H * N;
    const i64 tok0 = (i64)bb * T * C + hh * N;
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const int nchunks = T / L;
    float* ck = ck_ ? ck_ + (i64)(bb * H + hh) * nchunks * N * N : nullptr;
    const bf16* src[3] = {r_, k_, v_};

    // state tiles: S[nt] = rows row0+g / row0+g+8, columns 8nt+2t, 8nt+2t+1
    float S[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
            S[nt][e] = load_s0(s0_, s0_kind, sbase + (row0 + g + ((e & 2) ? 8 : 0)) * N + nt * 8 + 2 * t + (e & 1));

    const int lrow = tid >> 3, lseg = tid & 7;
    auto issue_loads = [&](int c, int stage) {
        const i64 off = tok0 + (i64)(c * L + lrow) * C + lseg * 8;
#pragma unroll
        for (int x = STATES_ONLY ? 1 : 0; x < 3; ++x) cp_async16(raw + ((stage * 3 + x) * L + lrow) * N + lseg * 8, src[x] + off);
        cp_async_commit();
    };
    // thread = (channel j, half of the chunk) in the preparation; its log-decays come straight from
    // global memory, one chunk ahead, in log2 units
    const int pj = tid & 63, phf = tid >> 6, pt0 = phf * 8;
    const float pu = __bfloat162float(u_[hh * N + pj]);
    uint32_t ldb[8];
    auto fetch_decay = [&](int c) {
#pragma unroll
        for (int q = 0; q < 8; ++q) ldb[q] = decay_bits<WMODE>(w_, tok0 + (i64)(c * L + pt0 + q) * C + pj, hh * N + pj);
    };
    issue_loads(0, 0);
    fetch_decay(0);

    for (int c = 0; c < nchunks; ++c) {
        const int stage = c & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (c + 1 < nchunks) issue_loads(c + 1, stage ^ 1);
        const bf16* R = raw + (stage * 3 + 0) * L * N;
        const bf16* K = raw + (stage * 3 + 1) * L * N;
        const bf16* V = raw + (stage * 3 + 2) * L * N;

        // ---- prep -----------------------------------------------------------------------------
        {
            float cs[8];
            float run = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) { run += decay_log2<WMODE>(ldb[q]); cs[q] = run; }
            Hs[phf * N + pj] = run;
            float xr[8], xk[8], xv[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                xr[q] = STATES_ONLY ? 0.f : to_f(R[(pt0 + q) * N + pj]);
                xk[q] = to_f(K[(pt0 + q) * N + pj]); xv[q] = to_f(V[(pt0 + q) * N + pj]);
            }
            __syncthreads();
            const float base = phf ? Hs[pj] : 0.f;
            const float total = Hs[pj] + Hs[N + pj];
            if (phf == 0) {
                We[pj] = fex2(total);
                if (-total > kMaxChunkLog2Decay)   // this (batch, head) unit must be redone by the general-shape kernel
                    atomicOr(unsafe_ + (((bb / flag_div) * H + hh) & (kChunkedFlagUnits - 1)), 1);
            }
            const int jp = (pj & ~7) + perm8(pj & 7);
            float pprev = phf ? fex2(base) : 1.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int tt = pt0 + q;
                const float lam = base + cs[q];
                const float p = fex2(lam), ip = fex2(-lam);
                Kt[tt * PK + jp] = tf32rf(xk[q] * ip);
                Vf[tt * PK + jp] = xv[q];
                if (!STATES_ONLY) {
                    Rt[tt * PK + jp] = tf32rf(xr[q] * pprev);
                    Ru[tt * PK + jp] = tf32rf(xr[q] * pu);
                    Kr[tt * PK + jp] = xk[q];
                }
                pprev = p;
            }
        }
        __syncthreads();
        if (c + 1 < nchunks) fetch_decay(c + 1);

        // ---- A: warp 0 the strict part k~_s.r~_t, warp 1 the diagonal sum_j r u k; stored [t][s] ----
        if (!STATES_ONLY && warp < 2) {
            const float* Am = warp ? Kr : Kt;
            const float* Bm = warp ? Ru : Rt;
            uint32_t areg[8][4];
            load_a_plain<8>(areg, Am, PK, 0, g, t);
            float U[2][4] = {};
            gemm_rs_plain<2, 8>(U, areg, Bm, PK, g, t);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int s = g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                    if (warp == 0) { if (s != tt) AT[tt * PU + s] = tf32rf(s < tt ? U[nt][e] : 0.f); }
                    else if (s == tt) AT[tt * PU + s] = tf32rf(U[nt][e]);
                }
        }

        // ---- X = S0 R~ --------------------------------------------------------------------------
        float X[2][4] = {};
#pragma unroll
        for (int ks = 0; ks < (STATES_ONLY ? 0 : 8); ++ks) {
            const uint32_t a0 = tf32r(S[ks][0]), a1 = tf32r(S[ks][2]), a2 = tf32r(S[ks][1]), a3 = tf32r(S[ks][3]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float* pr = Rt + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(X[nt], a0, a1, a2, a3, __float_as_uint(pr[0]), __float_as_uint(pr[4]));
            }
        }
        if (ck != nullptr) {  // state at the start of this chunk
            float* dst = ck + (i64)c * N * N;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                *reinterpret_cast<float2*>(dst + (row0 + g) * N + nt * 8 + 2 * t) = make_float2(S[nt][0], S[nt][1]);
                *reinterpret_cast<float2*>(dst + (row0 + g + 8) * N + nt * 8 + 2 * t) = make_float2(S[nt][2], S[nt][3]);
            }
        }
        if (!STATES_ONLY) __syncthreads();

        // ---- Y = X + V A;  S = (S + V K~) diag(We) ------------------------------------------------
        uint32_t vreg[2][4];
        load_a_kperm<2>(vreg, Vf, PK, row0, g, t);           // A[m=i][k=s] = v_s[i]
        if (!STATES_ONLY) gemm_rs<2, 2>(X, vreg, AT, PU, g, t);   // (B[k=s][n=t] = A[s][t])
        gemm_rs_kperm<8, 2>(S, vreg, Kt, PK, g, t);           // (B[k=t][n=j] = k~_t[j])
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float2 we = *reinterpret_cast<const float2*>(We + nt * 8 + 2 * t);
            S[nt][0] *= we.x; S[nt][1] *= we.y; S[nt][2] *= we.x; S[nt][3] *= we.y;
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                if (!STATES_ONLY) y_[tok0 + (i64)(c * L + tt) * C + i] = __float2bfloat16_rn(X[nt][e]);
            }
    }

    if (sT_ != nullptr) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<float2*>(sT_ + sbase + (row0 + g) * N + nt * 8 + 2 * t) = make_float2(S[nt][0], S[nt][1]);
            *reinterpret_cast<float2*>(sT_ + sbase + (row0 + g + 8) * N + nt * 8 + 2 * t) = make_float2(S[nt][2], S[nt][3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Backward.  Walks the chunks in reverse with E = dL/dS (rows = value i) and its transpose ET (rows =
// key j) as accumulator tiles; S0 (the state at the start of the chunk) comes from the checkpoints a
// forward pass of wkv6c_forward_kernel wrote.  With dY = [gy_t], Ew = E diag(We):
//   An[s,t] = A[s,t] (s < t), An[t,t] = beta_t = sum_j r_t u k_t          dV  = Ew K~^T + dY An^T
//   M = V^T dY:  G[s,t] = M[s,t] (s < t),  gamma_t = M[t,t]
//   dK' = We (E^T V) + R~^T G^T        dk_t = dK'[:,t] / P_t     + gamma_t u r_t
//   dR' = S0^T dY   + K~^T G           dr_t = dR'[:,t] * P_{t-1} + gamma_t u k_t
//   gu  = sum_t gamma_t r_t k_t
//   E  <- Ew + dY R~    (and the same for ET, transposed)
// Decay gradient, anchored at every chunk: with c_t = r_t drs_t - k_t dks_t (the parts of dr, dk without
// the u terms) and A0[j] = sum_i E_start[i,j] S0[i,j]:   dL/dlog w_t = A0 - sum_{tau<t} c_tau - r_t drs_t,
// and gw = dL/dlog w_t * log w_t (the derivative of log w = -exp(w_raw) by w_raw; wkv6_cuda_v1.cu:203).
struct BSmem {                                                       // floats
    static constexpr int kRawBytes = 2 * 4 * L * RP * 2;             // bf16 [2][4][L][RP]: r k v gy
    static constexpr int kS0 = kRawBytes / 4;                        // fp32 [N][PS0]
    static constexpr int kRt = kS0 + N * 68;                         // token-major, pitch PK, channels permuted:
    static constexpr int kKt = kRt + L * PK;
    static constexpr int kVf = kKt + L * PK;
    static constexpr int kDy = kVf + L * PK;
    static constexpr int kRu = kDy + L * PK;
    static constexpr int kKr = kRu + L * PK;
    static constexpr int kPt = kKr + L * PK;                         // P_t [t][j], natural order
    static constexpr int kLg = kPt + L * PK;                         // log w_t [t][j], natural order
    static constexpr int kAn = kLg + L * PK;                         // An [s][t]
    static constexpr int kGn = kAn + L * PU;                         // G  [s][t]
    static constexpr int kGt = kGn + L * PU;                         // G  [t][s]
    static constexpr int kGam = kGt + L * PU;                        // gamma [16]
    static constexpr int kWe = kGam + L;
    static constexpr int kHalf = kWe + N;
    static constexpr int kEnd = kHalf + 2 * N;
    static constexpr int kBytes = kEnd * 4;
};
constexpr int PS0 = 68;

__device__ __forceinline__ void store_ds0(void* p, int kind, i64 idx, float x) {
    if (kind == 2) reinterpret_cast<float*>(p)[idx] = x;
    else if (kind == 1) reinterpret_cast<bf16*>(p)[idx] = __float2bfloat16_rn(x);
}

template <int WMODE>
__global__ void __launch_bounds__(NT, 2)
wkv6c_backward_kernel(int T, int H, const bf16* __restrict__ r_, const bf16* __restrict__ k_,
                      const bf16* __restrict__ v_, const void* __restrict__ w_, const bf16* __restrict__ u_,
                      const bf16* __restrict__ gy_, const float* __restrict__ dsT_, const float* __restrict__ ck_,
                      bf16* __restrict__ gr_, bf16* __restrict__ gk_, bf16* __restrict__ gv_, bf16* __restrict__ gw_,
                      bf16* __restrict__ gu_, void* __restrict__ ds0_, int ds0_kind, float* __restrict__ gw32_,
                      float* __restrict__ gu32_) {
    constexpr bool gw_reduce = WMODE >= 2;   // a static decay has one gradient per channel and batch row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* sm = reinterpret_cast<float*>(smem_raw);
    bf16* raw = reinterpret_cast<bf16*>(smem_raw);
    float* S0s = sm + BSmem::kS0;
    float *Rt = sm + BSmem::kRt, *Kt = sm + BSmem::kKt, *Vf = sm + BSmem::kVf, *dYf = sm + BSmem::kDy;
    float *Ru = sm + BSmem::kRu, *Kr = sm + BSmem::kKr, *Pt = sm + BSmem::kPt, *Lg = sm + BSmem::kLg;
    float *An = sm + BSmem::kAn, *Gn = sm + BSmem::kGn, *Gt = sm + BSmem::kGt, *Gam = sm + BSmem::kGam;
    float *We = sm + BSmem::kWe, *Hs = sm + BSmem::kHalf;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = warp * 16;
    const int C = H * N;
    const i64 tok0 = (i64)bb * T * C + hh * N;
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const int nchunks = T / L;
    const float* ck = ck_ + (i64)(bb * H + hh) * nchunks * N * N;
    const bf16* src[4] = {r_, k_, v_, gy_};

    // E[nt]: rows i = row0+g / +8, cols j = 8nt+2t (+1).  ET[nt]: rows j = row0+g / +8, cols i = 8nt+2t (+1).
    float E[8][4], ET[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = row0 + g + ((e & 2) ? 8 : 0), col = nt * 8 + 2 * t + (e & 1);
            E[nt][e] = dsT_ ? dsT_[sbase + row * N + key_real(col)] : 0.f;      // E columns: logical key index
            ET[nt][e] = dsT_ ? dsT_[sbase + col * N + key_real(row)] : 0.f;    // ET rows: logical key index
        }
    // fragment rows (g, g+8) are the adjacent real key channels (2g, 2g+1) (key_logical / key_real)
    const float2 u01 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(u_ + hh * N + row0 + 2 * g));
    const float u0 = u01.x, u1 = u01.y;
    float gu_acc[2] = {0.f, 0.f}, gw_acc[2] = {0.f, 0.f};   // per-batch sums over time (gw only for a static decay)

    const int lrow = tid >> 3, lseg = tid & 7;
    auto issue_raw = [&](int c, int stage) {
        const i64 off = tok0 + (i64)(c * L + lrow) * C + lseg * 8;
#pragma unroll
        for (int x = 0; x < 4; ++x) cp_async16(raw + ((stage * 4 + x) * L + lrow) * RP + lseg * 8, src[x] + off);
        cp_async_commit();
    };
    auto issue_state = [&](int c) {
        const float* s0g = ck + (i64)c * N * N;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int idx = q * NT + tid, row = idx >> 4, seg = idx & 15;
            cp_async16(S0s + row * PS0 + seg * 4, s0g + row * N + seg * 4);
        }
        cp_async_commit();
    };
    const int pj = tid & 63, phf = tid >> 6, pt0 = phf * 8;
    const float pu = __bfloat162float(u_[hh * N + pj]);
    uint32_t ldb[8];   // decay inputs of this thread's (channel, 8 tokens) of the next chunk
    auto fetch_decay = [&](int c) {
#pragma unroll
        for (int q = 0; q < 8; ++q) ldb[q] = decay_bits<WMODE>(w_, tok0 + (i64)(c * L + pt0 + q) * C + pj, hh * N + pj);
    };
    issue_raw(nchunks - 1, (nchunks - 1) & 1);
    issue_state(nchunks - 1);
    fetch_decay(nchunks - 1);

    for (int c = nchunks - 1; c >= 0; --c) {
        const int stage = c & 1;
        cp_async_wait<1>();   // this chunk's input tiles (the state group may still be in flight)
        __syncthreads();
        if (c > 0) issue_raw(c - 1, stage ^ 1); else cp_async_commit();
        const bf16* R = raw + (stage * 4 + 0) * L * RP;
        const bf16* K = raw + (stage * 4 + 1) * L * RP;
        const bf16* V = raw + (stage * 4 + 2) * L * RP;
        const bf16* DY = raw + (stage * 4 + 3) * L * RP;
        const float* S0 = S0s;

        // ---- prep: thread = (channel, half of the chunk) ----------------------------------------
        {
            float cs[8], ld[8];
            float run = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) { ld[q] = decay_log2<WMODE>(ldb[q]); run += ld[q]; cs[q] = run; }
            float xr[8], xk[8], xv[8], xd[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                xr[q] = to_f(R[(pt0 + q) * RP + pj]); xk[q] = to_f(K[(pt0 + q) * RP + pj]);
                xv[q] = to_f(V[(pt0 + q) * RP + pj]); xd[q] = to_f(DY[(pt0 + q) * RP + pj]);
            }
            Hs[phf * N + pj] = run;
            __syncthreads();
            const float base = phf ? Hs[pj] : 0.f;
            const int jl = key_logical(pj);
            if (phf == 0) We[jl] = fex2(Hs[pj] + Hs[N + pj]);
            const int jp = (jl & ~7) + perm8(jl & 7);     // key-indexed arrays: logical order
            const int vp = (pj & ~7) + perm8(pj & 7);     // value-indexed arrays (v, gy): natural order
            float pprev = phf ? fex2(base) : 1.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int tt = pt0 + q;
                const float lam = base + cs[q];
                const float p = fex2(lam), ip = fex2(-lam);
                Rt[tt * PK + jp] = tf32rf(xr[q] * pprev);
                Kt[tt * PK + jp] = tf32rf(xk[q] * ip);
                Vf[tt * PK + vp] = xv[q];
                dYf[tt * PK + vp] = xd[q];
                Ru[tt * PK + jp] = tf32rf(xr[q] * pu);
                Kr[tt * PK + jp] = xk[q];
                Pt[tt * PK + pj] = p;
                Lg[tt * PK + pj] = ld[q] * 0.6931471805599453f;
                pprev = p;
            }
        }
        __syncthreads();
        if (c > 0) fetch_decay(c - 1);

        // ---- 16x16 matrices: warp 0 A (strict), warp 1 its diagonal beta, warp 2 M = V^T dY ---------
        if (warp < 3) {
            const float* Am = warp == 0 ? Kt : warp == 1 ? Kr : Vf;
            const float* Bm = warp == 0 ? Rt : warp == 1 ? Ru : dYf;
            uint32_t areg[8][4];
            load_a_plain<8>(areg, Am, PK, 0, g, t);
            float U[2][4] = {};
            gemm_rs_plain<2, 8>(U, areg, Bm, PK, g, t);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int s = g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                    if (warp == 0) { if (s != tt) An[s * PU + tt] = tf32rf(s < tt ? U[nt][e] : 0.f); }
                    else if (warp == 1) { if (s == tt) An[s * PU + tt] = tf32rf(U[nt][e]); }
                    else {
                        const float gval = tf32rf(s < tt ? U[nt][e] : 0.f);
                        Gn[s * PU + tt] = gval;
                        Gt[tt * PU + s] = gval;
                        if (s == tt) Gam[tt] = U[nt][e];
                    }
                }
        }

        // ---- Ew = E diag(We), ETw = diag(We) ET;  X2 = Ew K~^T -----------------------------------
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float2 we = *reinterpret_cast<const float2*>(We + nt * 8 + 2 * t);
            E[nt][0] *= we.x; E[nt][1] *= we.y; E[nt][2] *= we.x; E[nt][3] *= we.y;
        }
        {
            const float we0 = We[row0 + g], we1 = We[row0 + g + 8];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) { ET[nt][0] *= we0; ET[nt][1] *= we0; ET[nt][2] *= we1; ET[nt][3] *= we1; }
        }
        float X2[2][4] = {};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a0 = tf32r(E[ks][0]), a1 = tf32r(E[ks][2]), a2 = tf32r(E[ks][1]), a3 = tf32r(E[ks][3]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float* pk = Kt + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(X2[nt], a0, a1, a2, a3, __float_as_uint(pk[0]), __float_as_uint(pk[4]));
            }
        }
        cp_async_wait<1>();   // the chunk-start state has landed (only the next input tiles may be pending)
        __syncthreads();

        // ---- dV = Ew K~^T + dY An^T ---------------------------------------------------------------
        uint32_t dyreg[2][4];
        load_a_kperm<2>(dyreg, dYf, PK, row0, g, t);         // A[m=i][k=t] = dy_t[i]
        gemm_rs<2, 2>(X2, dyreg, An, PU, g, t);              // (B[k=t][n=s] = An[s][t])
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                gv_[tok0 + (i64)(c * L + tt) * C + i] = __float2bfloat16_rn(X2[nt][e]);
            }

        // ---- Z1 = ETw V,  Z2 = S0^T dY   (rows = key j) --------------------------------------------
        float Z1[2][4] = {}, Z2[2][4] = {};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a0 = tf32r(ET[ks][0]), a1 = tf32r(ET[ks][2]), a2 = tf32r(ET[ks][1]), a3 = tf32r(ET[ks][3]);
            const float* p0 = S0 + (ks * 8 + 2 * t) * PS0 + row0 + 2 * g;   // A[m=j][k=i] = S0[i][j], rows (g, g+8) = real (2g, 2g+1)
            const float2 sx = *reinterpret_cast<const float2*>(p0), sy = *reinterpret_cast<const float2*>(p0 + PS0);
            const uint32_t s0a = tf32r(sx.x), s1a = tf32r(sx.y), s2a = tf32r(sy.x), s3a = tf32r(sy.y);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float* pv = Vf + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z1[nt], a0, a1, a2, a3, __float_as_uint(pv[0]), __float_as_uint(pv[4]));
                const float* pd = dYf + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z2[nt], s0a, s1a, s2a, s3a, __float_as_uint(pd[0]), __float_as_uint(pd[4]));
            }
        }

        // ---- dK' += R~^T G^T,  dR' += K~^T G: scaled vectors as hi + lo TF32 pairs ------------------
        uint32_t rthi[2][4];
        {
            uint32_t rtlo[2][4], kthi[2][4], ktlo[2][4];
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                float2 pp2 = make_float2(1.f, 1.f);
                if (ks > 0 || t > 0) pp2 = *reinterpret_cast<const float2*>(Pt + (ks * 8 + 2 * t - 1) * PK + row0 + 2 * g);
#pragma unroll
                for (int uh = 0; uh < 2; ++uh) {      // fragment slots e = 2*uh (row g) and 2*uh+1 (row g+8) = real channels 2g, 2g+1
                    const int u = ks * 8 + 2 * t + uh, jr = row0 + 2 * g;
                    const float2 pu2 = *reinterpret_cast<const float2*>(Pt + u * PK + jr);
                    const float2 r2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(R + u * RP + jr));
                    const float2 k2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(K + u * RP + jr));
                    const float xr[2] = {r2.x * pp2.x, r2.y * pp2.y}, xk[2] = {k2.x * frcp(pu2.x), k2.y * frcp(pu2.y)};
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int e = 2 * uh + h;
                        rthi[ks][e] = tf32(xr[h]); rtlo[ks][e] = tf32r(xr[h] - __uint_as_float(rthi[ks][e]));
                        kthi[ks][e] = tf32(xk[h]); ktlo[ks][e] = tf32r(xk[h] - __uint_as_float(kthi[ks][e]));
                    }
                    pp2 = pu2;
                }
            }
            gemm_rs2<2, 2>(Z1, rthi, rtlo, Gn, PU, g, t);     // (B[k=t][n=s] = G[s][t])
            gemm_rs2<2, 2>(Z2, kthi, ktlo, Gt, PU, g, t);     // (B[k=s][n=t] = G[s][t])
        }

        // ---- E and ET updates ----------------------------------------------------------------------
        gemm_rs_kperm<8, 2>(E, dyreg, Rt, PK, g, t);          // E  += dY R~      (B[k=t][n=j] = r~_t[j])
        gemm_rs_kperm<8, 2>(ET, rthi, dYf, PK, g, t);         // ET += R~^T dY^T  (B[k=t][n=i] = dy_t[i])

        float A0[2] = {0.f, 0.f};                             // sum_i E_start[i,j] S0[i,j]
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int q = 0; q < 2; ++q) {         // ET rows (g, g+8) = real key channels (2g, 2g+1)
                const float2 sv = *reinterpret_cast<const float2*>(S0 + (nt * 8 + 2 * t + q) * PS0 + row0 + 2 * g);
                A0[0] = fmaf(ET[nt][q], sv.x, A0[0]);
                A0[1] = fmaf(ET[nt][2 + q], sv.y, A0[1]);
            }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            A0[h2] += __shfl_xor_sync(0xffffffffu, A0[h2], 1);
            A0[h2] += __shfl_xor_sync(0xffffffffu, A0[h2], 2);
        }
        __syncthreads();      // every warp is done with the staged state
        if (c > 0) issue_state(c - 1); else cp_async_commit();

        // ---- per-token gradients, rows j = row0+g (+8), columns = tokens ----------------------------
        float cterm[2][4], rdr[2][4], lw[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int q = 0; q < 2; ++q) {         // token tt, both rows of the thread: real channels jr, jr+1
                const int tt = nt * 8 + 2 * t + q, jr = row0 + 2 * g;
                const float2 p2 = *reinterpret_cast<const float2*>(Pt + tt * PK + jr);
                float2 pp2 = make_float2(1.f, 1.f);
                if (tt > 0) pp2 = *reinterpret_cast<const float2*>(Pt + (tt - 1) * PK + jr);
                const float2 lg2 = *reinterpret_cast<const float2*>(Lg + tt * PK + jr);
                const float2 r2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(R + tt * RP + jr));
                const float2 k2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(K + tt * RP + jr));
                const float pv[2] = {p2.x, p2.y}, ppv[2] = {pp2.x, pp2.y}, lgv[2] = {lg2.x, lg2.y};
                const float rv[2] = {r2.x, r2.y}, kv[2] = {k2.x, k2.y}, uv[2] = {u0, u1};
                const float gam = Gam[tt];
                float dk[2], dr[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int e = 2 * h + q;
                    const float dks = Z1[nt][e] * frcp(pv[h]), drs = Z2[nt][e] * ppv[h];
                    const float gu_ = gam * uv[h];
                    dk[h] = fmaf(gu_, rv[h], dks);
                    dr[h] = fmaf(gu_, kv[h], drs);
                    gu_acc[h] = fmaf(gam, rv[h] * kv[h], gu_acc[h]);
                    rdr[nt][e] = rv[h] * drs;
                    cterm[nt][e] = rdr[nt][e] - kv[h] * dks;
                    lw[nt][e] = lgv[h];
                }
                const i64 o = tok0 + (i64)(c * L + tt) * C + jr;
                *reinterpret_cast<uint32_t*>(gk_ + o) = f2_to_bf16x2(dk[0], dk[1]);
                *reinterpret_cast<uint32_t*>(gr_ + o) = f2_to_bf16x2(dr[0], dr[1]);
            }
        // exclusive prefix of cterm along the 16 tokens of each row: lanes t = 0..3 of a quad hold
        // tokens (2t, 2t+1) of tile 0 and (8+2t, 8+2t+1) of tile 1
        float Gw[2][4];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const int e0 = h2 * 2;
            const float p0 = cterm[0][e0] + cterm[0][e0 + 1], p1 = cterm[1][e0] + cterm[1][e0 + 1];
            float i0 = p0, i1 = p1;                          // inclusive scans over the quad
            float n0 = __shfl_up_sync(0xffffffffu, i0, 1, 4), n1 = __shfl_up_sync(0xffffffffu, i1, 1, 4);
            if (t >= 1) { i0 += n0; i1 += n1; }
            n0 = __shfl_up_sync(0xffffffffu, i0, 2, 4); n1 = __shfl_up_sync(0xffffffffu, i1, 2, 4);
            if (t >= 2) { i0 += n0; i1 += n1; }
            const float tot0 = __shfl_sync(0xffffffffu, i0, 3, 4);
            const float ex0 = i0 - p0, ex1 = tot0 + i1 - p1;
            const float pre[4] = {ex0, ex0 + cterm[0][e0], ex1, ex1 + cterm[1][e0]};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int nt = q >> 1, e = e0 + (q & 1);
                Gw[h2][q] = (A0[h2] - pre[q] - rdr[nt][e]) * lw[nt][e];
            }
        }
        if (gw_reduce) {
#pragma unroll
            for (int q = 0; q < 4; ++q) { gw_acc[0] += Gw[0][q]; gw_acc[1] += Gw[1][q]; }
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int tt = (q >> 1) * 8 + 2 * t + (q & 1);
                *reinterpret_cast<uint32_t*>(gw_ + tok0 + (i64)(c * L + tt) * C + row0 + 2 * g) = f2_to_bf16x2(Gw[0][q], Gw[1][q]);
            }
        }
    }

    // gu: this thread holds the sums over its tokens; the four lanes of a quad share a row
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        gu_acc[h2] += __shfl_xor_sync(0xffffffffu, gu_acc[h2], 1);
        gu_acc[h2] += __shfl_xor_sync(0xffffffffu, gu_acc[h2], 2);
        if (t == 0) gu_[(i64)bb * C + hh * N + row0 + 2 * g + h2] = __float2bfloat16_rn(gu_acc[h2]);
        if (t == 0 && gu32_ != nullptr) gu32_[(i64)bb * C + hh * N + row0 + 2 * g + h2] = gu_acc[h2];   // unrounded
        if (gw_reduce) {
            gw_acc[h2] += __shfl_xor_sync(0xffffffffu, gw_acc[h2], 1);
            gw_acc[h2] += __shfl_xor_sync(0xffffffffu, gw_acc[h2], 2);
            if (t == 0) gw_[(i64)bb * C + hh * N + row0 + 2 * g + h2] = __float2bfloat16_rn(gw_acc[h2]);
            if (t == 0 && gw32_ != nullptr) gw32_[(i64)bb * C + hh * N + row0 + 2 * g + h2] = gw_acc[h2];
        }
    }
    if (ds0_kind != 0) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                store_ds0(ds0_, ds0_kind, sbase + (row0 + g + ((e & 2) ? 8 : 0)) * N + key_real(nt * 8 + 2 * t + (e & 1)), E[nt][e]);
    }
}

}  // namespace v6c

// Flags of the chunked kernels ("a chunk's decay was too strong"), one per (batch, head) unit (unit index
// modulo kChunkedFlagUnits: units that share a flag are redone together).  A call enqueues: clear the flags, the
// chunked kernels (which may raise some), the general-shape kernel (whose thread blocks read theirs and redo only
// the flagged units).  On one stream that is ordered, so every (device, stream) pair owns one slot for good and
// calls on different streams never share one.  The table holds 256 pairs per process; beyond that the function returns NULL and the caller runs
// the general-shape kernel alone.  (A CUDA graph captured from such a call carries the slot of the
// capturing stream: replay it on one stream at a time.)
constexpr int kFlagSlots = 256;
static __device__ int g_chunked_unsafe[kFlagSlots * kChunkedFlagUnits];
int* wkv6_chunked_flag(cudaStream_t st) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int* base[kMaxDevices] = {};             // device address of the slot array, per device
    static struct { int dev; cudaStream_t st; } owner[kFlagSlots];
    static int used = 0;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (base[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_chunked_unsafe) != cudaSuccess) return nullptr;
        base[dev] = static_cast<int*>(p);
    }
    for (int i = 0; i < used; ++i)
        if (owner[i].dev == dev && owner[i].st == st) return base[dev] + i * kChunkedFlagUnits;
    if (used == kFlagSlots) return nullptr;
    owner[used].dev = dev;
    owner[used].st = st;
    return base[dev] + (used++) * kChunkedFlagUnits;
}

static std::atomic<int> g_wkv6_forward_tcgen05{1}, g_wkv6_backward_tcgen05{1};
void wkv6_select_forward(int tcgen05) { g_wkv6_forward_tcgen05.store(tcgen05 ? 1 : 0); }
void wkv6_select_backward(int tcgen05) { g_wkv6_backward_tcgen05.store(tcgen05 ? 1 : 0); }
int wkv6_forward_choice() { return g_wkv6_forward_tcgen05.load(); }

int wkv6_chunked_forward(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode,
                         const void* u, const void* s0, int s0_kind, void* y, float* sT, float* ck, int* unsafe,
                         cudaStream_t st, int flag_div) {
    using namespace v6c;
    // a forward that leaves no chunk states for a backward pass: the tcgen05 kernel where it can run
    if (y != nullptr && ck == nullptr && unsafe != nullptr && g_wkv6_forward_tcgen05.load()) {
        const int rc = wkv6_l32_forward(B, T, H, r, k, v, w, w_mode, u, s0, s0_kind, y, sT, nullptr, unsafe, st, flag_div);
        if (rc != 1) return rc;
    }
    RWKV_REQUIRE(w_mode >= 0 && w_mode <= 3, RWKVB200_EINVAL, "wkv6_forward(chunked): decay mode %d", w_mode);
    dim3 grid(H, B);
#define RWKV_GO1(M, SO)                                                                                                \
    do {                                                                                                               \
        cudaError_t e = cudaFuncSetAttribute(wkv6c_forward_kernel<M, SO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             FSmem::kBytes);                                                           \
        RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv6_forward: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        wkv6c_forward_kernel<M, SO><<<grid, NT, FSmem::kBytes, st>>>(T, H, (const bf16*)r, (const bf16*)k, (const bf16*)v, \
                                                                     w, (const bf16*)u, s0, s0_kind, (bf16*)y, sT, ck,  \
                                                                     unsafe, flag_div);                                \
    } while (0)
#define RWKV_GO(M)                    \
    do {                              \
        if (y == nullptr) RWKV_GO1(M, true); \
        else RWKV_GO1(M, false);      \
    } while (0)
    switch (w_mode) {
        case 0: RWKV_GO(0); break;
        case 1: RWKV_GO(1); break;
        case 2: RWKV_GO(2); break;
        default: RWKV_GO(3); break;
    }
#undef RWKV_GO
#undef RWKV_GO1
    return check_launch("wkv6_forward(chunked)");
}

// The backward with its pass that rebuilds the chunk-start states into `ck` (the caller's scratch buffer): on the
// tcgen05 kernels (32-token chunks) where they can run, else on the mma.sync kernels (16-token chunks).
int wkv6_backward_with_states(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode,
                              const void* u, const void* s0, int s0_kind, const void* gy, const float* dsT, float* ck, void* gr,
                              void* gk, void* gv, void* gw, void* gu, void* ds0, int ds0_kind, int* unsafe, cudaStream_t st,
                              float* gw32, float* gu32) {
    if (unsafe != nullptr && g_wkv6_backward_tcgen05.load()) {
        const int rc = wkv6_l32_forward(B, T, H, r, k, v, w, w_mode, u, s0, s0_kind, nullptr, nullptr, ck, unsafe, st, 1);
        if (rc != 1) {
            if (rc != 0) return rc;
            return wkv6_l32_backward(B, T, H, r, k, v, w, w_mode, u, gy, dsT, ck, gr, gk, gv, gw, gu, ds0, ds0_kind, st, gw32, gu32);
        }
    }
    if (int e = wkv6_chunked_forward(B, T, H, r, k, v, w, w_mode, u, s0, s0_kind, nullptr, nullptr, ck, unsafe, st)) return e;
    return wkv6_chunked_backward(B, T, H, r, k, v, w, w_mode, u, gy, dsT, ck, gr, gk, gv, gw, gu, ds0, ds0_kind, st, gw32, gu32);
}

int wkv6_chunked_backward(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode,
                          const void* u, const void* gy, const float* dsT, const float* ck, void* gr, void* gk,
                          void* gv, void* gw, void* gu, void* ds0, int ds0_kind, cudaStream_t st, float* gw32,
                          float* gu32) {
    using namespace v6c;
    static_assert(BSmem::kBytes <= 113 * 1024, "backward shared memory must allow 2 CTAs per SM");
    RWKV_REQUIRE(w_mode >= 0 && w_mode <= 3, RWKVB200_EINVAL, "wkv6_backward(chunked): decay mode %d", w_mode);
    dim3 grid(H, B);
#define RWKV_GO(M)                                                                                                      \
    do {                                                                                                                \
        cudaError_t e = cudaFuncSetAttribute(wkv6c_backward_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                             BSmem::kBytes);                                                            \
        RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv6_backward: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
        wkv6c_backward_kernel<M><<<grid, NT, BSmem::kBytes, st>>>(T, H, (const bf16*)r, (const bf16*)k, (const bf16*)v, w, \
                                                                  (const bf16*)u, (const bf16*)gy, dsT, ck, (bf16*)gr,  \
                                                                  (bf16*)gk, (bf16*)gv, (bf16*)gw, (bf16*)gu, ds0,      \
                                                                  ds0_kind, gw32, gu32);                                \
    } while (0)
    switch (w_mode) {
        case 0: RWKV_GO(0); break;
        case 1: RWKV_GO(1); break;
        case 2: RWKV_GO(2); break;
        default: RWKV_GO(3); break;
    }
#undef RWKV_GO
    return check_launch("wkv6_backward(chunked)");
}

}  // namespace rwkvb200
