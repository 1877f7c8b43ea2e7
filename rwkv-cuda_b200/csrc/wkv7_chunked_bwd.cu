// RWKV-7 backward, head size 64, bf16 activations: chunked tensor-core kernel.
//
// Walks the chunks of 16 tokens in reverse.  Carried across chunks, in registers as MMA
// accumulator tiles, are E = dL/dS (rows = value i) and its transpose ET (rows = key j), warp w
// holding rows 16w..16w+15 of each.  With the scaled operands of wkv7_chunked.cuh, S0 the saved
// state at the start of the chunk, SA the saved sa vectors, Ew = E diag(We):
//   EV  = (Ew B~^T + dY U_br^T) T^T                         e_t = E_t b_t  (64 x 16)
//   dV  =  Ew K~^T + EV U_ak^T + dY U_kr^T
//   P1 = EV^T V (u>t)   P2 = dY^T V (u>=t)   P3 = EV^T SA (u>t)   P4 = dY^T SA (u>=t)      (16 x 16)
//   dK' = We (E^T V)  + A~^T P1 + R~^T P2        dk_t = dK'[:,t] / W_t
//   dB' = We (E^T SA) + A~^T P3 + R~^T P4        db_t = dB'[:,t] / W_t
//   dA' = S0^T EV + B~^T P3^T + K~^T P1^T        da_t = dA'[:,t] * W_{t-1}
//   dR' = S0^T dY + B~^T P4^T + K~^T P2^T        dr_t = dR'[:,t] * W_t
//   E  <- Ew + EV A~ + dY R~        (and the same for ET, transposed)
// The decay gradient needs no second pass over state pairs: with c_t = r dr + a da - b db - k dk
// (per key channel) and A0[j] = sum_i E_start[i,j] S0[i,j],
//   dL/dlog d_t = A0 - sum_{tau<t} c_tau - a_t da_t
// anchored afresh at every chunk so rounding does not accumulate along the sequence.
#include "wkv7_chunked.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7c {

constexpr int PS0 = 68;  // pitch of the staged 64x64 state (read along its rows' index)

struct BwdSmem {
    static constexpr int kRawBytes = 2 * 7 * L * RP * 2;             // bf16 [2][7][L*N]: r w k v a b dy
    static constexpr int kSa = kRawBytes / 4;                        // fp32 [L][PT]
    static constexpr int kS0 = kSa + L * PT;                         // fp32 [N][PS0]
    static constexpr int kAt = kS0 + N * PS0;                        // token-major, pitch PK, channels permuted:
    static constexpr int kRt = kAt + L * PK;
    static constexpr int kBt = kRt + L * PK;
    static constexpr int kKt = kBt + L * PK;
    static constexpr int kVf = kKt + L * PK;                         // v, dy as fp32
    static constexpr int kDy = kVf + L * PK;
    static constexpr int kEv = kDy + L * PK;                         // EV [t][i]
    static constexpr int kWt = kEv + L * PK;                         // W_t [t][j], natural order
    static constexpr int kU = kWt + L * PK;                          // Uab Uak Ubr Ukr T (natural [s][t])
    static constexpr int kP = kU + 5 * L * PU;                       // P1..P4 natural, then transposed
    static constexpr int kWe = kP + 8 * L * PU;
    static constexpr int kHalf = kWe + N;
    static constexpr int kEnd = kHalf + 2 * N;
    static constexpr int kBytes = kEnd * 4;
};

__device__ __forceinline__ void store_bf16(bf16* p, float x) { *p = __float2bfloat16_rn(x); }

__global__ void __launch_bounds__(NT, 2)
wkv7c_backward_kernel(int T, int H, const bf16* __restrict__ r_, const bf16* __restrict__ w_,
                      const bf16* __restrict__ k_, const bf16* __restrict__ v_, const bf16* __restrict__ a_,
                      const bf16* __restrict__ b_, const bf16* __restrict__ dy_, const float* __restrict__ dsT_,
                      const float* __restrict__ ck_, const float* __restrict__ sa_, float* __restrict__ ds0_,
                      bf16* __restrict__ dr_, bf16* __restrict__ dw_, bf16* __restrict__ dk_, bf16* __restrict__ dv_,
                      bf16* __restrict__ da_, bf16* __restrict__ db_) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* sm = reinterpret_cast<float*>(smem_raw);
    bf16* raw = reinterpret_cast<bf16*>(smem_raw);
    float *SAs = sm + BwdSmem::kSa, *S0s = sm + BwdSmem::kS0;
    float *At = sm + BwdSmem::kAt, *Rt = sm + BwdSmem::kRt, *Bt = sm + BwdSmem::kBt, *Kt = sm + BwdSmem::kKt;
    float *Vf = sm + BwdSmem::kVf, *dYf = sm + BwdSmem::kDy, *EVs = sm + BwdSmem::kEv;
    float* Wt = sm + BwdSmem::kWt;
    float *Uab = sm + BwdSmem::kU, *Uak = Uab + L * PU, *Ubr = Uak + L * PU, *Ukr = Ubr + L * PU, *Tn = Ukr + L * PU;
    float *Pn = sm + BwdSmem::kP, *Ptr = Pn + 4 * L * PU;   // natural / transposed, index 0..3 = P1..P4
    float *We = sm + BwdSmem::kWe, *Hs = sm + BwdSmem::kHalf;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = warp * 16;
    const int C = H * N;
    const i64 tok0 = (i64)bb * T * C + hh * N;
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const int nchunks = T / L;
    const float* ck = ck_ + (i64)(bb * H + hh) * nchunks * N * N;
    const bf16* src[7] = {r_, w_, k_, v_, a_, b_, dy_};

    // E[nt]: rows i = row0+g / +8, cols j = 8nt+2t (+1).  ET[nt]: rows j = row0+g / +8, cols i = 8nt+2t (+1).
    float E[8][4], ET[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = row0 + g + ((e & 2) ? 8 : 0), col = nt * 8 + 2 * t + (e & 1);
            E[nt][e] = dsT_ ? dsT_[sbase + row * N + col] : 0.f;
            ET[nt][e] = dsT_ ? dsT_[sbase + col * N + row] : 0.f;
        }

    const int lrow = tid >> 3, lseg = tid & 7;
    auto issue_raw = [&](int c, int stage) {
        const i64 off = tok0 + (i64)(c * L + lrow) * C + lseg * 8;
#pragma unroll
        for (int x = 0; x < 7; ++x) cp_async16(raw + ((stage * 7 + x) * L + lrow) * RP + lseg * 8, src[x] + off);
        cp_async_commit();
    };
    // sa (16 x 64 fp32) and the chunk-start state (64 x 64 fp32) are single-buffered: they are
    // requested as soon as the previous chunk has finished with the buffers
    auto issue_state = [&](int c) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int idx = tid * 2 + q, row = idx >> 4, seg = idx & 15;
            cp_async16(SAs + row * PT + seg * 4, sa_ + tok0 + (i64)(c * L + row) * C + seg * 4);
        }
        const float* s0g = ck + (i64)c * N * N;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int idx = q * NT + tid, row = idx >> 4, seg = idx & 15;
            cp_async16(S0s + row * PS0 + seg * 4, s0g + row * N + seg * 4);
        }
        cp_async_commit();
    };
    issue_raw(nchunks - 1, (nchunks - 1) & 1);
    issue_state(nchunks - 1);

    for (int c = nchunks - 1; c >= 0; --c) {
        const int stage = c & 1;
        cp_async_wait<1>();   // this chunk's input tiles (the state group may still be in flight)
        __syncthreads();
        if (c > 0) issue_raw(c - 1, stage ^ 1); else cp_async_commit();
        const bf16* R = raw + (stage * 7 + 0) * L * RP;
        const bf16* Wr = raw + (stage * 7 + 1) * L * RP;
        const bf16* K = raw + (stage * 7 + 2) * L * RP;
        const bf16* V = raw + (stage * 7 + 3) * L * RP;
        const bf16* A = raw + (stage * 7 + 4) * L * RP;
        const bf16* Bv = raw + (stage * 7 + 5) * L * RP;
        const bf16* DY = raw + (stage * 7 + 6) * L * RP;
        const float* SA = SAs;
        const float* S0 = S0s;

        // ---- prep -----------------------------------------------------------------------------
        {
            const int j = tid & 63, hf = tid >> 6, t0 = hf * 8;
            float cs[8];
            float run = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float x = to_f(Wr[(t0 + q) * RP + j]);
                run += __fdividef(kWScale, 1.f + __expf(-x));
                cs[q] = run;
            }
            Hs[hf * N + j] = run;
            __syncthreads();
            const float base = hf ? Hs[j] : 0.f;
            if (hf == 0) We[j] = __expf(Hs[j] + Hs[N + j]);
            float wprev = hf ? __expf(base) : 1.f;
            const int jp = (j & ~7) + perm8(j & 7);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int tt = t0 + q;
                const float lam = base + cs[q];
                const float wt = __expf(lam), iw = __expf(-lam);
                At[tt * PK + jp] = tf32f(to_f(A[tt * RP + j]) * wprev);
                Rt[tt * PK + jp] = tf32f(to_f(R[tt * RP + j]) * wt);
                Bt[tt * PK + jp] = tf32f(to_f(Bv[tt * RP + j]) * iw);
                Kt[tt * PK + jp] = tf32f(to_f(K[tt * RP + j]) * iw);
                Vf[tt * PK + jp] = to_f(V[tt * RP + j]);
                dYf[tt * PK + jp] = to_f(DY[tt * RP + j]);
                Wt[tt * PK + j] = wt;
                wprev = wt;
            }
        }
        __syncthreads();

        // ---- small products: warp 0 U_ab (+T), 1 U_ak, 2 U_br, 3 U_kr; stored as [s][t] --------
        {
            const float* Am = (warp & 1) ? Kt : Bt;
            const float* Bm = (warp & 2) ? Rt : At;
            uint32_t areg[8][4];
            load_a_plain<8>(areg, Am, PK, 0, g, t);
            float U[2][4] = {};
            gemm_rs_plain<2, 8>(U, areg, Bm, PK, g, t);
            float* dst = Uab + warp * L * PU;
            const bool strict = warp < 2;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int s = g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                    const bool keep = strict ? (s < tt) : (s <= tt);
                    const float val = keep ? U[nt][e] : 0.f;
                    dst[s * PU + tt] = warp == 0 ? val : tf32f(val);
                }
            if (warp == 0) {
                __syncwarp();
                tri_inverse<true>(Uab, Tn, lane);
            }
        }

        // ---- Ew = E diag(We), ETw = diag(We) ET;  X2 = Ew [B~ | K~]^T -------------------------
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
        float X2[4][4] = {};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a0 = tf32(E[ks][0]), a1 = tf32(E[ks][2]), a2 = tf32(E[ks][1]), a3 = tf32(E[ks][3]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float* pb = Bt + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(X2[nt], a0, a1, a2, a3, __float_as_uint(pb[0]), __float_as_uint(pb[4]));
                const float* pk = Kt + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(X2[2 + nt], a0, a1, a2, a3, __float_as_uint(pk[0]), __float_as_uint(pk[4]));
            }
        }
        cp_async_wait<1>();   // sa and the chunk-start state have landed (only the next input tiles may be pending)
        __syncthreads();

        // ---- EV and dV ------------------------------------------------------------------------
        {   // sa arrived as fp32: round it to TF32 once (it is only ever an MMA operand here)
            float4* p = reinterpret_cast<float4*>(SAs + lrow * PT + lseg * 8);
            float4 x0 = p[0], x1 = p[1];
            x0.x = tf32f(x0.x); x0.y = tf32f(x0.y); x0.z = tf32f(x0.z); x0.w = tf32f(x0.w);
            x1.x = tf32f(x1.x); x1.y = tf32f(x1.y); x1.z = tf32f(x1.z); x1.w = tf32f(x1.w);
            p[0] = x0; p[1] = x1;
        }
        uint32_t dyreg[2][4], xreg[2][4], evreg[2][4];
        load_a_kperm<2>(dyreg, dYf, PK, row0, g, t);         // A[m=i][k=u] = dy_u[i]
        gemm_rs<2, 2>(X2, dyreg, Ubr, PU, g, t);             // += dY U_br^T   (B[k=u][n=t] = U_br[t][u])
        acc_to_a<2>(xreg, X2);
        float EV[2][4] = {};
        gemm_rs<2, 2>(EV, xreg, Tn, PU, g, t);               // EV = (.) T^T   (B[k=u][n=t] = T[t][u])
        acc_to_a<2>(evreg, EV);
        gemm_rs<2, 2>(X2 + 2, evreg, Uak, PU, g, t);         // dV = Ew K~^T + EV U_ak^T + dY U_kr^T
        gemm_rs<2, 2>(X2 + 2, dyreg, Ukr, PU, g, t);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                store_bf16(dv_ + tok0 + (i64)(c * L + tt) * C + i, X2[2 + nt][e]);
                EVs[tt * PK + (i & ~7) + perm8(i & 7)] = tf32f(EV[nt][e]);
            }
        __syncthreads();

        // ---- Gram blocks: warp 0 P1 = EV^T V, 1 P3 = EV^T SA, 2 P2 = dY^T V, 3 P4 = dY^T SA ----
        {
            const float* Am = (warp & 2) ? dYf : EVs;
            const float* Bm = (warp & 1) ? SA : Vf;
            uint32_t areg[8][4];
            load_a_plain<8>(areg, Am, PK, 0, g, t);
            float P[2][4] = {};
            if (warp & 1) gemm_rs<2, 8>(P, areg, Bm, PT, g, t);        // sa: natural order, 64-bit reads
            else gemm_rs_plain<2, 8>(P, areg, Bm, PK, g, t);
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
        // ---- Z1 = ETw [V | SA],  Z2 = S0^T [EV | dY]   (rows = key j) ---------------------------
        float Z1[4][4] = {}, Z2[4][4] = {};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a0 = tf32(ET[ks][0]), a1 = tf32(ET[ks][2]), a2 = tf32(ET[ks][1]), a3 = tf32(ET[ks][3]);
            const float* p0 = S0 + (ks * 8 + 2 * t) * PS0 + row0 + g;   // A[m=j][k=i] = S0[i][j]
            const uint32_t s0a = tf32(p0[0]), s1a = tf32(p0[8]), s2a = tf32(p0[PS0]), s3a = tf32(p0[PS0 + 8]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float* pv = Vf + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z1[nt], a0, a1, a2, a3, __float_as_uint(pv[0]), __float_as_uint(pv[4]));
                const uint2 bs = lds2(SA + (nt * 8 + g) * PT + ks * 8 + 2 * t);
                mma8(Z1[2 + nt], a0, a1, a2, a3, bs.x, bs.y);
                const float* pe = EVs + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z2[nt], s0a, s1a, s2a, s3a, __float_as_uint(pe[0]), __float_as_uint(pe[4]));
                const float* pd = dYf + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z2[2 + nt], s0a, s1a, s2a, s3a, __float_as_uint(pd[0]), __float_as_uint(pd[4]));
            }
        }
        __syncthreads();

        // ---- dK' dB' (in Z1) and dA' dR' (in Z2) ------------------------------------------------
        // The scaled vectors enter these last small products unrounded (hi + lo TF32 parts, two MMAs):
        // their rounding error is what the decay gradient's running sum would otherwise amplify.
        uint32_t atreg[2][4], rtreg[2][4], btreg[2][4], ktreg[2][4];
        uint32_t atlo[2][4], rtlo[2][4], btlo[2][4], ktlo[2][4];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int u = ks * 8 + 2 * t + (e >> 1), j = row0 + g + (e & 1) * 8;
                const float wu = Wt[u * PK + j], iwu = __frcp_rn(wu);
                const float wp = u > 0 ? Wt[(u - 1) * PK + j] : 1.f;
                const float xa = to_f(A[u * RP + j]) * wp, xr = to_f(R[u * RP + j]) * wu;
                const float xb = to_f(Bv[u * RP + j]) * iwu, xk = to_f(K[u * RP + j]) * iwu;
                atreg[ks][e] = tf32(xa); atlo[ks][e] = tf32(xa - __uint_as_float(atreg[ks][e]));
                rtreg[ks][e] = tf32(xr); rtlo[ks][e] = tf32(xr - __uint_as_float(rtreg[ks][e]));
                btreg[ks][e] = tf32(xb); btlo[ks][e] = tf32(xb - __uint_as_float(btreg[ks][e]));
                ktreg[ks][e] = tf32(xk); ktlo[ks][e] = tf32(xk - __uint_as_float(ktreg[ks][e]));
            }
        const float *P1n = Pn, *P2n = Pn + L * PU, *P3n = Pn + 2 * L * PU, *P4n = Pn + 3 * L * PU;
        const float *P1t = Ptr, *P2t = Ptr + L * PU, *P3t = Ptr + 2 * L * PU, *P4t = Ptr + 3 * L * PU;
        gemm_rs2<2, 2>(Z1, atreg, atlo, P1t, PU, g, t);      // dK' += A~^T P1 + R~^T P2  (B[k=u][n=t] = P[u][t])
        gemm_rs2<2, 2>(Z1, rtreg, rtlo, P2t, PU, g, t);
        gemm_rs2<2, 2>(Z1 + 2, atreg, atlo, P3t, PU, g, t);  // dB'
        gemm_rs2<2, 2>(Z1 + 2, rtreg, rtlo, P4t, PU, g, t);
        gemm_rs2<2, 2>(Z2, btreg, btlo, P3n, PU, g, t);      // dA' += B~^T P3^T + K~^T P1^T (B[k=s][n=t] = P[t][s])
        gemm_rs2<2, 2>(Z2, ktreg, ktlo, P1n, PU, g, t);
        gemm_rs2<2, 2>(Z2 + 2, btreg, btlo, P4n, PU, g, t);  // dR'
        gemm_rs2<2, 2>(Z2 + 2, ktreg, ktlo, P2n, PU, g, t);

        // ---- E and ET updates ------------------------------------------------------------------
        gemm_rs_kperm<8, 2>(E, evreg, At, PK, g, t);         // E += EV A~   (B[k=t][n=j] = a~_t[j])
        gemm_rs_kperm<8, 2>(E, dyreg, Rt, PK, g, t);         //    + dY R~
        gemm_rs_kperm<8, 2>(ET, atreg, EVs, PK, g, t);       // ET += A~^T EV^T (B[k=t][n=i] = e_t[i])
        gemm_rs_kperm<8, 2>(ET, rtreg, dYf, PK, g, t);       //     + R~^T dY^T

        // ---- per-token gradients, rows j = row0+g (+8), columns = tokens --------------------------
        float A0[2] = {0.f, 0.f};                            // sum_i E_start[i,j] S0[i,j]
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = row0 + g + ((e & 2) ? 8 : 0), i = nt * 8 + 2 * t + (e & 1);
                A0[e >> 1] = fmaf(ET[nt][e], S0[i * PS0 + j], A0[e >> 1]);
            }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            A0[h2] += __shfl_xor_sync(0xffffffffu, A0[h2], 1);
            A0[h2] += __shfl_xor_sync(0xffffffffu, A0[h2], 2);
        }
        __syncthreads();      // every warp is done with sa and the staged state
        if (c > 0) issue_state(c - 1); else cp_async_commit();
        float cterm[2][4], ada[2][4], sgd[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                const float wt = Wt[tt * PK + j], iw = __frcp_rn(wt);
                const float wprev = tt > 0 ? Wt[(tt - 1) * PK + j] : 1.f;
                const float dk = Z1[nt][e] * iw, db = Z1[2 + nt][e] * iw;
                const float da = Z2[nt][e] * wprev, dr = Z2[2 + nt][e] * wt;
                const float rr = to_f(R[tt * RP + j]), aa = to_f(A[tt * RP + j]);
                const float bq = to_f(Bv[tt * RP + j]), kq = to_f(K[tt * RP + j]);
                const i64 o = tok0 + (i64)(c * L + tt) * C + j;
                store_bf16(dk_ + o, dk); store_bf16(db_ + o, db); store_bf16(da_ + o, da); store_bf16(dr_ + o, dr);
                ada[nt][e] = aa * da;
                cterm[nt][e] = rr * dr + ada[nt][e] - bq * db - kq * dk;
                const float sg = 1.f / (1.f + __expf(-to_f(Wr[tt * RP + j])));
                sgd[nt][e] = kWScale * sg * (1.f - sg);
            }
        // exclusive prefix of cterm along the 16 tokens of each row: lanes t = 0..3 of a quad hold
        // tokens (2t, 2t+1) of tile 0 and (8+2t, 8+2t+1) of tile 1
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
            const int j = row0 + g + h2 * 8;
            const float pre[4] = {ex0, ex0 + cterm[0][e0], ex1, ex1 + cterm[1][e0]};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int nt = q >> 1, e = e0 + (q & 1), tt = nt * 8 + 2 * t + (q & 1);
                const float G = A0[h2] - pre[q] - ada[nt][e];
                store_bf16(dw_ + tok0 + (i64)(c * L + tt) * C + j, G * sgd[nt][e]);
            }
        }
    }

    if (ds0_ != nullptr) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<float2*>(ds0_ + sbase + (row0 + g) * N + nt * 8 + 2 * t) = make_float2(E[nt][0], E[nt][1]);
            *reinterpret_cast<float2*>(ds0_ + sbase + (row0 + g + 8) * N + nt * 8 + 2 * t) = make_float2(E[nt][2], E[nt][3]);
        }
    }
}

}  // namespace v7c

int wkv7_chunked_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v,
                          const void* a, const void* b, const void* dy, const float* dsT, const float* s,
                          const float* sa, float* ds0, void* dr, void* dw, void* dk, void* dv, void* da, void* db,
                          cudaStream_t st) {
    using namespace v7c;
    cudaError_t e = cudaFuncSetAttribute(wkv7c_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_backward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7c_backward_kernel<<<grid, NT, BwdSmem::kBytes, st>>>(
        T, H, (const bf16*)r, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b,
        (const bf16*)dy, dsT, s, sa, ds0, (bf16*)dr, (bf16*)dw, (bf16*)dk, (bf16*)dv, (bf16*)da, (bf16*)db);
    return check_launch("wkv7_backward(chunked)");
}

}  // namespace rwkvb200
