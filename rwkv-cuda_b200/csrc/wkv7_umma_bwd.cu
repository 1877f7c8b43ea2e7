// RWKV-7 backward, head size 64, bf16 activations: tcgen05 kernel.
//
// Same chunked algorithm as wkv7_chunked_bwd.cu (formulas in its header).  The two carried state
// gradients E (rows = value i) and ET (rows = key j) live in tensor memory for the whole
// sequence, and the products that read or update them run as tcgen05.mma (kind::tf32, M = 64):
//   U  = [B~;K~][A~|R~]^T     (K = 64)          X2 = Ew [B~|K~]^T  (A = E  from tensor memory)
//   Z1 = ETw [V|SA]           (A = ET)          E += [EV|dY][A~;R~],  ET += [A~;R~]^T [EV|dY]^T  (K = 32)
// The small K = 16 chains, the Gram blocks, S0^T [EV|dY] (whose A operand would have to be the
// transposed saved state) and the per-token epilogue stay on mma.sync in registers; tcgen05.ld of
// shape 16x256b hands accumulators over in the mma.sync fragment layout.  The saved chunk-start
// state is not staged in shared memory: each thread fetches exactly the 32 elements it needs, once,
// and uses them both as A fragments and for the anchor sum of the decay gradient.
//
//   tensor memory (256 columns): E [0,64)  ET [64,128)  X2 [128,160)  Z1 [160,192)  U [192,224)
#include "wkv7_umma.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7u {

constexpr int kBwdTmemCols = 256;
constexpr int kColE = 0, kColET = 64, kColX2 = 128, kColZ1 = 160, kColUb = 192;

__device__ int g_umma_bwd_error = 0;

struct BSmem {
    static constexpr int kRawBytes = 2 * 7 * L * RP * 2;         // bf16 [2][7][L*N]: r w k v a b dy
    static constexpr int kARt = kRawBytes;                        // [A~;R~]  token-major, K = j
    static constexpr int kBKt = kARt + 16 * LBO_T;                // [B~;K~]  (read as 64 rows: runs on into VSt)
    static constexpr int kVSt = kBKt + 16 * LBO_T;                // [V;SA]   token-major, K = i
    static constexpr int kARc = kVSt + 16 * LBO_T;                // [a~|r~]  by key channel j,   K = token (32)
    static constexpr int kEDc = kARc + 8 * LBO_C;                 // [EV|dY]  by value channel i, K = token (32)
    static constexpr int kEVs = kEDc + 8 * LBO_C;                 // EV, dY as [token][channel], pitch PK, channels permuted
    static constexpr int kDYf = kEVs + L * PK * 4;
    static constexpr int kWt = kDYf + L * PK * 4;                 // W_t [t][j]
    static constexpr int kU = kWt + L * PK * 4;                   // Uab Uak Ubr Ukr T, natural [s][t]
    static constexpr int kP = kU + 5 * L * PU * 4;                // P1..P4 natural, then transposed
    static constexpr int kWe = kP + 8 * L * PU * 4;
    static constexpr int kHalf = kWe + N * 4;
    static constexpr int kBar = kHalf + 2 * N * 4;                // 3 mbarriers + tmem slot
    static constexpr int kBytes = kBar + 48;
};
static_assert(BSmem::kBytes <= 113 * 1024, "backward shared memory must allow 2 CTAs per SM");

__device__ __forceinline__ void store_bf16(bf16* p, float x) { *p = __float2bfloat16_rn(x); }

__global__ void __launch_bounds__(NT, 2)
wkv7u_backward_kernel(int T, int H, const bf16* __restrict__ r_, const bf16* __restrict__ w_,
                      const bf16* __restrict__ k_, const bf16* __restrict__ v_, const bf16* __restrict__ a_,
                      const bf16* __restrict__ b_, const bf16* __restrict__ dy_, const float* __restrict__ dsT_,
                      const float* __restrict__ ck_, const float* __restrict__ sa_, float* __restrict__ ds0_,
                      bf16* __restrict__ dr_, bf16* __restrict__ dw_, bf16* __restrict__ dk_, bf16* __restrict__ dv_,
                      bf16* __restrict__ da_, bf16* __restrict__ db_) {
    extern __shared__ __align__(128) unsigned char smem[];
    bf16* raw = reinterpret_cast<bf16*>(smem);
    unsigned char *ARt = smem + BSmem::kARt, *BKt = smem + BSmem::kBKt, *VSt = smem + BSmem::kVSt;
    unsigned char *ARc = smem + BSmem::kARc, *EDc = smem + BSmem::kEDc;
    float *EVs = reinterpret_cast<float*>(smem + BSmem::kEVs), *dYf = reinterpret_cast<float*>(smem + BSmem::kDYf);
    float* Wt = reinterpret_cast<float*>(smem + BSmem::kWt);
    float* Um = reinterpret_cast<float*>(smem + BSmem::kU);
    float *Uab = Um, *Uak = Um + L * PU, *Ubr = Um + 2 * L * PU, *Ukr = Um + 3 * L * PU, *Tn = Um + 4 * L * PU;
    float *Pn = reinterpret_cast<float*>(smem + BSmem::kP), *Ptr = Pn + 4 * L * PU;
    float* We = reinterpret_cast<float*>(smem + BSmem::kWe);
    float* Hs = reinterpret_cast<float*>(smem + BSmem::kHalf);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + BSmem::kBar);   // [0] U   [1] X2,Z1   [2] E,ET updates
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 3);

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = warp * 16;
    const int C = H * N;
    const i64 tok0 = (i64)bb * T * C + hh * N;
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const int nchunks = T / L;
    const float* ck = ck_ + (i64)(bb * H + hh) * nchunks * N * N;
    const bf16* src[7] = {r_, w_, k_, v_, a_, b_, dy_};

    if (tid == 0) {
#pragma unroll
        for (int q = 0; q < 3; ++q) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar + q)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(kBwdTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tw = tmem + ((uint32_t)(warp * 32) << 16);

    // E = dsT (rows i), ET = dsT^T (rows j) -> tensor memory
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        float e[4], et[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int row = row0 + g + ((q & 2) ? 8 : 0), col = nt * 8 + 2 * t + (q & 1);
            e[q] = dsT_ ? dsT_[sbase + row * N + col] : 0.f;
            et[q] = dsT_ ? dsT_[sbase + col * N + row] : 0.f;
        }
        tmem_st8(tw + kColE + nt * 8, e);
        tmem_st8(tw + kColET + nt * 8, et);
    }
    tmem_wait_st();

    const int lrow = tid >> 3, lseg = tid & 7;
    auto issue_raw = [&](int c, int stage) {
        const i64 off = tok0 + (i64)(c * L + lrow) * C + lseg * 8;
#pragma unroll
        for (int x = 0; x < 7; ++x) cp_async16(raw + ((stage * 7 + x) * L + lrow) * RP + lseg * 8, src[x] + off);
        cp_async_commit();
    };
    // sa (16 tokens x 64 fp32) goes straight into rows 16..31 of the [V;SA] operand, 16 bytes a piece
    auto issue_sa = [&](int c) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int idx = tid * 2 + q, row = idx >> 4, seg = idx & 15;
            cp_async16(VSt + canon(16 + row, seg * 4, LBO_T), sa_ + tok0 + (i64)(c * L + row) * C + seg * 4);
        }
        cp_async_commit();
    };
    issue_raw(nchunks - 1, (nchunks - 1) & 1);
    issue_sa(nchunks - 1);
    int fail = 0;

    WKV7_PHASE_BEGIN();
    for (int c = nchunks - 1; c >= 0; --c) {
        const int stage = c & 1;
        const uint32_t par = (nchunks - 1 - c) & 1;
        cp_async_wait<1>();
        tc_fence_before();
        if (__syncthreads_or(fail)) break;
        tc_fence_after();
        if (c > 0) issue_raw(c - 1, stage ^ 1); else cp_async_commit();
        const bf16* R = raw + (stage * 7 + 0) * L * RP;
        const bf16* Wr = raw + (stage * 7 + 1) * L * RP;
        const bf16* K = raw + (stage * 7 + 2) * L * RP;
        const bf16* V = raw + (stage * 7 + 3) * L * RP;
        const bf16* A = raw + (stage * 7 + 4) * L * RP;
        const bf16* Bv = raw + (stage * 7 + 5) * L * RP;
        const bf16* DY = raw + (stage * 7 + 6) * L * RP;

        WKV7_PHASE(0);   // wait for input tiles
        // the 32 elements of the chunk-start state this thread needs: S0[i = 8ks+2t (+1)][j = row0+g (+8)]
        float s0f[8][4];
        {
            const float* s0g = ck + (i64)c * N * N + row0 + g;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const float* p0 = s0g + (ks * 8 + 2 * t) * N;
                s0f[ks][0] = __ldg(p0); s0f[ks][1] = __ldg(p0 + 8); s0f[ks][2] = __ldg(p0 + N); s0f[ks][3] = __ldg(p0 + N + 8);
            }
        }

        // ---- prep -----------------------------------------------------------------------------
        {
            const int j = tid & 63, hf = tid >> 6, t0 = hf * 8;
            float cs[8];
            float run = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float x = to_f(Wr[(t0 + q) * RP + j]);
                run = fmaf(kWScale2, frcp(1.f + fexp(-x)), run);
                cs[q] = run;
            }
            Hs[hf * N + j] = run;
            __syncthreads();
            const float base = hf ? Hs[j] : 0.f;
            if (hf == 0) We[j] = fex2(Hs[j] + Hs[N + j]);
            float wprev = hf ? fex2(base) : 1.f;
            const int jp = (j & ~7) + perm8(j & 7);
            float at[8], rt[8], dyv[8];
            // loads of a batch of four tokens before its stores (tiles and operand arrays share one
            // shared-memory block: the compiler keeps a load behind every earlier store)
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                float xb[4], xk[4], xv[4], wt[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int tt = t0 + 4 * hb + q, qq = 4 * hb + q;
                    const float lam = base + cs[qq];
                    wt[q] = fex2(lam);
                    const float iw = fex2(-lam);
                    at[qq] = tf32f(to_f(A[tt * RP + j]) * wprev);
                    rt[qq] = tf32f(to_f(R[tt * RP + j]) * wt[q]);
                    dyv[qq] = to_f(DY[tt * RP + j]);
                    xb[q] = tf32f(to_f(Bv[tt * RP + j]) * iw);
                    xk[q] = tf32f(to_f(K[tt * RP + j]) * iw);
                    xv[q] = to_f(V[tt * RP + j]);
                    wprev = wt[q];
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int tt = t0 + 4 * hb + q, qq = 4 * hb + q;
                    *reinterpret_cast<float*>(ARt + canon(tt, j, LBO_T)) = at[qq];
                    *reinterpret_cast<float*>(ARt + canon(16 + tt, j, LBO_T)) = rt[qq];
                    *reinterpret_cast<float*>(BKt + canon(tt, j, LBO_T)) = xb[q];
                    *reinterpret_cast<float*>(BKt + canon(16 + tt, j, LBO_T)) = xk[q];
                    *reinterpret_cast<float*>(VSt + canon(tt, j, LBO_T)) = xv[q];
                    dYf[tt * PK + jp] = dyv[qq];
                    Wt[tt * PK + j] = wt[q];
                }
            }
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {
                *reinterpret_cast<float4*>(ARc + canon(j, t0 + 4 * q4, LBO_C)) = make_float4(at[4 * q4], at[4 * q4 + 1], at[4 * q4 + 2], at[4 * q4 + 3]);
                *reinterpret_cast<float4*>(ARc + canon(j, 16 + t0 + 4 * q4, LBO_C)) = make_float4(rt[4 * q4], rt[4 * q4 + 1], rt[4 * q4 + 2], rt[4 * q4 + 3]);
                *reinterpret_cast<float4*>(EDc + canon(j, 16 + t0 + 4 * q4, LBO_C)) = make_float4(dyv[4 * q4], dyv[4 * q4 + 1], dyv[4 * q4 + 2], dyv[4 * q4 + 3]);
            }
        }
        cp_async_wait<1>();   // sa of this chunk has landed (only the next input tiles may still be in flight)
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();

        WKV7_PHASE(1);   // prep + barrier
        // ---- U on the tensor core; meanwhile round sa and scale E, ET by We -----------------------
        if (tid == 0) {
            const uint32_t id32 = umma_idesc(32);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                umma_ss(tmem + kColUb, umma_desc(smem_u32(BKt) + ks * 2 * LBO_T, LBO_T),
                        umma_desc(smem_u32(ARt) + ks * 2 * LBO_T, LBO_T), id32, ks > 0);
            umma_commit(bar);
        }
        {   // sa arrived as fp32: round it to TF32 in place (two 16-byte pieces per thread)
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int idx = tid * 2 + q, row = idx >> 4, seg = idx & 15;
                float4* p = reinterpret_cast<float4*>(VSt + canon(16 + row, seg * 4, LBO_T));
                float4 x = *p;
                x.x = tf32f(x.x); x.y = tf32f(x.y); x.z = tf32f(x.z); x.w = tf32f(x.w);
                *p = x;
            }
        }
        {
            float Ed[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) tmem_ld8(Ed[nt], tw + kColE + nt * 8);
            tmem_wait_ld();
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float2 we = *reinterpret_cast<const float2*>(We + nt * 8 + 2 * t);
                Ed[nt][0] *= we.x; Ed[nt][1] *= we.y; Ed[nt][2] *= we.x; Ed[nt][3] *= we.y;
                tmem_st8(tw + kColE + nt * 8, Ed[nt]);
            }
            const float we0 = We[row0 + g], we1 = We[row0 + g + 8];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) tmem_ld8(Ed[nt], tw + kColET + nt * 8);
            tmem_wait_ld();
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                Ed[nt][0] *= we0; Ed[nt][1] *= we0; Ed[nt][2] *= we1; Ed[nt][3] *= we1;
                tmem_st8(tw + kColET + nt * 8, Ed[nt]);
            }
            tmem_wait_st();
        }
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();

        WKV7_PHASE(2);   // sa rounding, E/ET scaling, barrier
        // ---- X2 = Ew [B~|K~]^T and Z1 = ETw [V|SA] on the tensor core -----------------------------
        if (tid == 0) {
            const uint32_t id32 = umma_idesc(32);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                umma_ts(tmem + kColX2, tmem + kColE + ks * 8, umma_desc(smem_u32(BKt) + ks * 2 * LBO_T, LBO_T), id32, ks > 0);
                umma_ts(tmem + kColZ1, tmem + kColET + ks * 8, umma_desc(smem_u32(VSt) + ks * 2 * LBO_T, LBO_T), id32, ks > 0);
            }
            umma_commit(bar + 1);
        }
        if (!mbar_wait(bar, par)) fail = 1;
        tc_fence_after();
        if (warp < 2) {   // warp 0: rows b~ -> U_ab, U_br;  warp 1: rows k~ -> U_ak, U_kr;  all stored [s][t]
            float U[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) tmem_ld8(U[nt], tw + kColUb + nt * 8);
            tmem_wait_ld();
            float* dstA = warp == 0 ? Uab : Uak;
            float* dstR = warp == 0 ? Ubr : Ukr;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int s = g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                    const float ua = s < tt ? U[nt][e] : 0.f, ur = s <= tt ? U[2 + nt][e] : 0.f;
                    dstA[s * PU + tt] = warp == 0 ? ua : tf32f(ua);
                    dstR[s * PU + tt] = tf32f(ur);
                }
            if (warp == 0) {
                __syncwarp();
                tri_inverse<true>(Uab, Tn, lane);
            }
        }
        WKV7_PHASE(3);   // U wait, extraction, inverse
        if (!mbar_wait(bar + 1, par)) fail = 2;
        tc_fence_after();
        float X2[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) tmem_ld8(X2[nt], tw + kColX2 + nt * 8);
        tmem_wait_ld();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();

        WKV7_PHASE(4);   // X2 wait, barrier
        // ---- EV and dV (mma.sync, registers) --------------------------------------------------------
        uint32_t dyreg[2][4], xreg[2][4], evreg[2][4];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {   // A[m=i][k=u] = dy_u[i] from the by-channel operand (K index 16+u)
            const int u = 16 + ks * 8 + 2 * t;
            dyreg[ks][0] = *reinterpret_cast<const uint32_t*>(EDc + canon(row0 + g, u, LBO_C));
            dyreg[ks][1] = *reinterpret_cast<const uint32_t*>(EDc + canon(row0 + g + 8, u, LBO_C));
            dyreg[ks][2] = *reinterpret_cast<const uint32_t*>(EDc + canon(row0 + g, u + 1, LBO_C));
            dyreg[ks][3] = *reinterpret_cast<const uint32_t*>(EDc + canon(row0 + g + 8, u + 1, LBO_C));
        }
        gemm_rs<2, 2>(X2, dyreg, Ubr, PU, g, t);             // += dY U_br^T
        acc_to_a<2>(xreg, X2);
        float EV[2][4] = {};
        gemm_rs<2, 2>(EV, xreg, Tn, PU, g, t);               // EV = (.) T^T
        acc_to_a<2>(evreg, EV);
        gemm_rs<2, 2>(X2 + 2, evreg, Uak, PU, g, t);         // dV = Ew K~^T + EV U_ak^T + dY U_kr^T
        gemm_rs<2, 2>(X2 + 2, dyreg, Ukr, PU, g, t);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int u = nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(EDc + canon(row0 + g, u, LBO_C)) = make_float2(__uint_as_float(evreg[nt][0]), __uint_as_float(evreg[nt][2]));
            *reinterpret_cast<float2*>(EDc + canon(row0 + g + 8, u, LBO_C)) = make_float2(__uint_as_float(evreg[nt][1]), __uint_as_float(evreg[nt][3]));
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                store_bf16(dv_ + tok0 + (i64)(c * L + tt) * C + i, X2[2 + nt][e]);
                EVs[tt * PK + (i & ~7) + perm8(i & 7)] = tf32f(EV[nt][e]);
            }
        }
        proxy_fence();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();

        WKV7_PHASE(5);   // EV chain, dV, barrier
        // ---- E += [EV|dY][A~;R~],  ET += [A~;R~]^T [EV|dY]^T on the tensor core -------------------
        if (tid == 0) {
            const uint32_t id64 = umma_idesc(64);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ed = umma_desc(smem_u32(EDc) + ks * 2 * LBO_C, LBO_C);
                const uint64_t ar = umma_desc(smem_u32(ARc) + ks * 2 * LBO_C, LBO_C);
                umma_ss(tmem + kColE, ed, ar, id64, 1);
                umma_ss(tmem + kColET, ar, ed, id64, 1);
            }
            umma_commit(bar + 2);
        }

        // ---- Gram blocks: warp 0 P1 = EV^T V, 1 P3 = EV^T SA, 2 P2 = dY^T V, 3 P4 = dY^T SA ----
        float P[2][4] = {};
        {
            const float* Am = (warp & 2) ? dYf : EVs;
            const int brow = (warp & 1) ? 16 : 0;            // rows of [V;SA]
            uint32_t areg[8][4];
            load_a_plain<8>(areg, Am, PK, 0, g, t);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const uint2 b2 = *reinterpret_cast<const uint2*>(VSt + canon(brow + nt * 8 + g, ks * 8 + 2 * t, LBO_T));
                    mma8(P[nt], areg[ks][0], areg[ks][1], areg[ks][2], areg[ks][3], b2.x, b2.y);
                }
        }
        WKV7_PHASE(6);   // Gram
        // ---- Z1 from tensor memory;  Z2 = S0^T [EV | dY]  (rows = key j) --------------------------
        float Z1[4][4], Z2[4][4] = {};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) tmem_ld8(Z1[nt], tw + kColZ1 + nt * 8);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t s0a = tf32(s0f[ks][0]), s1a = tf32(s0f[ks][1]), s2a = tf32(s0f[ks][2]), s3a = tf32(s0f[ks][3]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float* pe = EVs + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z2[nt], s0a, s1a, s2a, s3a, __float_as_uint(pe[0]), __float_as_uint(pe[4]));
                const float* pd = dYf + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z2[2 + nt], s0a, s1a, s2a, s3a, __float_as_uint(pd[0]), __float_as_uint(pd[4]));
            }
        }
        tmem_wait_ld();
        {   // the Gram blocks go to shared memory only now: stores placed earlier would hold back the loads of Z1/Z2 above
            const int which = (warp == 0) ? 0 : (warp == 2) ? 1 : (warp == 1) ? 2 : 3;  // P1 P2 P3 P4
            const bool strict = !(warp & 2);
            float* pn = Pn + which * L * PU;
            float* pt = Ptr + which * L * PU;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int u = g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                    const bool keep = strict ? (u > tt) : (u >= tt);
                    const float val = tf32f(keep ? P[nt][e] : 0.f);
                    pn[u * PU + tt] = val;
                    pt[tt * PU + u] = val;
                }
        }
        __syncthreads();

        WKV7_PHASE(7);   // Z2, barrier
        // ---- dK' dB' (in Z1) and dA' dR' (in Z2): scaled vectors as hi + lo TF32 pairs ---------------
        {
            uint32_t hi[2][4], lo[2][4], hi2[2][4], lo2[2][4];
            const float *P1n = Pn, *P2n = Pn + L * PU, *P3n = Pn + 2 * L * PU, *P4n = Pn + 3 * L * PU;
            const float *P1t = Ptr, *P2t = Ptr + L * PU, *P3t = Ptr + 2 * L * PU, *P4t = Ptr + 3 * L * PU;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int u = ks * 8 + 2 * t + (e >> 1), j = row0 + g + (e & 1) * 8;
                    const float wu = Wt[u * PK + j];
                    const float wp = u > 0 ? Wt[(u - 1) * PK + j] : 1.f;
                    const float xa = to_f(A[u * RP + j]) * wp, xr = to_f(R[u * RP + j]) * wu;
                    hi[ks][e] = tf32(xa); lo[ks][e] = tf32(xa - __uint_as_float(hi[ks][e]));
                    hi2[ks][e] = tf32(xr); lo2[ks][e] = tf32(xr - __uint_as_float(hi2[ks][e]));
                }
            gemm_rs2<2, 2>(Z1, hi, lo, P1t, PU, g, t);          // dK' += A~^T P1 + R~^T P2
            gemm_rs2<2, 2>(Z1, hi2, lo2, P2t, PU, g, t);
            gemm_rs2<2, 2>(Z1 + 2, hi, lo, P3t, PU, g, t);      // dB' += A~^T P3 + R~^T P4
            gemm_rs2<2, 2>(Z1 + 2, hi2, lo2, P4t, PU, g, t);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int u = ks * 8 + 2 * t + (e >> 1), j = row0 + g + (e & 1) * 8;
                    const float iwu = frcp(Wt[u * PK + j]);
                    const float xb = to_f(Bv[u * RP + j]) * iwu, xk = to_f(K[u * RP + j]) * iwu;
                    hi[ks][e] = tf32(xb); lo[ks][e] = tf32(xb - __uint_as_float(hi[ks][e]));
                    hi2[ks][e] = tf32(xk); lo2[ks][e] = tf32(xk - __uint_as_float(hi2[ks][e]));
                }
            gemm_rs2<2, 2>(Z2, hi, lo, P3n, PU, g, t);          // dA' += B~^T P3^T + K~^T P1^T
            gemm_rs2<2, 2>(Z2, hi2, lo2, P1n, PU, g, t);
            gemm_rs2<2, 2>(Z2 + 2, hi, lo, P4n, PU, g, t);      // dR' += B~^T P4^T + K~^T P2^T
            gemm_rs2<2, 2>(Z2 + 2, hi2, lo2, P2n, PU, g, t);
        }

        WKV7_PHASE(8);   // hi/lo loaders + P products
        // ---- anchor of the decay gradient: A0[j] = sum_i ET_start[j,i] S0[i,j] ------------------------
        if (!mbar_wait(bar + 2, par)) fail = 3;
        tc_fence_after();
        float A0[2] = {0.f, 0.f};
        {
            float Ed[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) tmem_ld8(Ed[nt], tw + kColET + nt * 8);
            tmem_wait_ld();
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                A0[0] = fmaf(Ed[nt][0], s0f[nt][0], fmaf(Ed[nt][1], s0f[nt][2], A0[0]));
                A0[1] = fmaf(Ed[nt][2], s0f[nt][1], fmaf(Ed[nt][3], s0f[nt][3], A0[1]));
            }
        }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            A0[h2] += __shfl_xor_sync(0xffffffffu, A0[h2], 1);
            A0[h2] += __shfl_xor_sync(0xffffffffu, A0[h2], 2);
        }
        if (c > 0) issue_sa(c - 1); else cp_async_commit();   // every reader of this chunk's sa is done

        WKV7_PHASE(9);   // wait E/ET update, A0
        // ---- per-token gradients, rows j = row0+g (+8), columns = tokens --------------------------
        float cterm[2][4], ada[2][4], sgd[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                const float wt = Wt[tt * PK + j], iw = frcp(wt);
                const float wprev = tt > 0 ? Wt[(tt - 1) * PK + j] : 1.f;
                const float dk = Z1[nt][e] * iw, db = Z1[2 + nt][e] * iw;
                const float da = Z2[nt][e] * wprev, dr = Z2[2 + nt][e] * wt;
                const float rr = to_f(R[tt * RP + j]), aa = to_f(A[tt * RP + j]);
                const float bq = to_f(Bv[tt * RP + j]), kq = to_f(K[tt * RP + j]);
                const i64 o = tok0 + (i64)(c * L + tt) * C + j;
                store_bf16(dk_ + o, dk); store_bf16(db_ + o, db); store_bf16(da_ + o, da); store_bf16(dr_ + o, dr);
                ada[nt][e] = aa * da;
                cterm[nt][e] = rr * dr + ada[nt][e] - bq * db - kq * dk;
                const float sg = frcp(1.f + fexp(-to_f(Wr[tt * RP + j])));
                sgd[nt][e] = kWScale * sg * (1.f - sg);
            }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const int e0 = h2 * 2;
            const float p0 = cterm[0][e0] + cterm[0][e0 + 1], p1 = cterm[1][e0] + cterm[1][e0 + 1];
            float i0 = p0, i1 = p1;
            float n0 = __shfl_up_sync(0xffffffffu, i0, 1, 4), n1 = __shfl_up_sync(0xffffffffu, i1, 1, 4);
            if (t >= 1) { i0 += n0; i1 += n1; }
            n0 = __shfl_up_sync(0xffffffffu, i0, 2, 4); n1 = __shfl_up_sync(0xffffffffu, i1, 2, 4);
            if (t >= 2) { i0 += n0; i1 += n1; }
            const float tot0 = __shfl_sync(0xffffffffu, i0, 3, 4);
            const float ex0 = i0 - p0, ex1 = tot0 + i1 - p1;
            const int j = row0 + g + h2 * 8;
            const float pre[4] = {ex0, ex0 + cterm[0][e0], ex1, ex1 + cterm[1][e0]};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int nt = q >> 1, e = e0 + (q & 1), tt = nt * 8 + 2 * t + (q & 1);
                const float G = A0[h2] - pre[q] - ada[nt][e];
                store_bf16(dw_ + tok0 + (i64)(c * L + tt) * C + j, G * sgd[nt][e]);
            }
        }
        WKV7_PHASE(10);  // per-token gradients
    }

    if (!fail && ds0_ != nullptr) {
        tc_fence_after();
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float e[4];
            tmem_ld8(e, tw + kColE + nt * 8);
            tmem_wait_ld();
            *reinterpret_cast<float2*>(ds0_ + sbase + (row0 + g) * N + nt * 8 + 2 * t) = make_float2(e[0], e[1]);
            *reinterpret_cast<float2*>(ds0_ + sbase + (row0 + g + 8) * N + nt * 8 + 2 * t) = make_float2(e[2], e[3]);
        }
    }
    if (fail && tid == 0) atomicMax(&g_umma_bwd_error, 10 + fail);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kBwdTmemCols) : "memory");
}

WKV7_PHASE_READER(rwkvb200_phase_clocks_umma_bwd)

}  // namespace v7u

int wkv7_umma_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v,
                       const void* a, const void* b, const void* dy, const float* dsT, const float* s,
                       const float* sa, float* ds0, void* dr, void* dw, void* dk, void* dv, void* da, void* db,
                       cudaStream_t st) {
    using namespace v7u;
    cudaError_t e = cudaFuncSetAttribute(wkv7u_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BSmem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_backward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7u_backward_kernel<<<grid, NT, BSmem::kBytes, st>>>(
        T, H, (const bf16*)r, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b,
        (const bf16*)dy, dsT, s, sa, ds0, (bf16*)dr, (bf16*)dw, (bf16*)dk, (bf16*)dv, (bf16*)da, (bf16*)db);
    return check_launch("wkv7_backward(tcgen05)");
}

int wkv7_umma_bwd_error() {
    int h = 0;
    cudaMemcpyFromSymbol(&h, v7u::g_umma_bwd_error, sizeof(int));
    return h;
}

}  // namespace rwkvb200
