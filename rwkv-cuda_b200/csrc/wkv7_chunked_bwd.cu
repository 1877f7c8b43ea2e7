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
// Key channels are handled under the relabelling of wkv7_chunked.cuh (key_logical / key_real):
// E columns, ET rows and every [t][j] operand array are in logical order, W_t, the staged state and
// the bf16 tiles in real order.
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
            E[nt][e] = dsT_ ? dsT_[sbase + row * N + key_real(col)] : 0.f;
            ET[nt][e] = dsT_ ? dsT_[sbase + col * N + key_real(row)] : 0.f;
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

    WKV7_PHASE_BEGIN();
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

        WKV7_PHASE(0);   // wait for input tiles
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
            WKV7_PHASE(14);  // prep: log-decays of the half chunk
            Hs[hf * N + j] = run;
            __syncthreads();
            const float base = hf ? Hs[j] : 0.f;
            const int jl = key_logical(j);
            if (hf == 0) We[jl] = fex2(Hs[j] + Hs[N + j]);
            float wprev = hf ? fex2(base) : 1.f;
            const int jp = (jl & ~7) + perm8(jl & 7);   // key-indexed arrays: logical order
            const int ip = (j & ~7) + perm8(j & 7);     // value-indexed arrays (v, dy): natural order
            // All loads of a batch of four tokens come before its stores: the staged tiles and the
            // operand arrays live in the same shared-memory block, so the compiler keeps every load
            // behind the stores that precede it in program order.
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                float xa[4], xr[4], xb[4], xk[4], xv[4], xd[4], wt[4], iw[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int tt = t0 + 4 * hb + q;
                    xa[q] = to_f(A[tt * RP + j]); xr[q] = to_f(R[tt * RP + j]); xb[q] = to_f(Bv[tt * RP + j]);
                    xk[q] = to_f(K[tt * RP + j]); xv[q] = to_f(V[tt * RP + j]); xd[q] = to_f(DY[tt * RP + j]);
                    const float lam = base + cs[4 * hb + q];
                    wt[q] = fex2(lam); iw[q] = fex2(-lam);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int tt = t0 + 4 * hb + q;
                    At[tt * PK + jp] = tf32rf(xa[q] * wprev);
                    Rt[tt * PK + jp] = tf32rf(xr[q] * wt[q]);
                    Bt[tt * PK + jp] = tf32rf(xb[q] * iw[q]);
                    Kt[tt * PK + jp] = tf32rf(xk[q] * iw[q]);
                    Vf[tt * PK + ip] = xv[q];
                    dYf[tt * PK + ip] = xd[q];
                    Wt[tt * PK + j] = wt[q];
                    wprev = wt[q];
                }
            }
        }
        WKV7_PHASE(15);  // prep: exchange barrier, scaled operands
        __syncthreads();

        WKV7_PHASE(1);   // prep
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
                    dst[s * PU + tt] = warp == 0 ? val : tf32rf(val);
                }
            if (warp == 0) {
                __syncwarp();
                tri_inverse<true>(Uab, Tn, lane);
            }
        }

        WKV7_PHASE(2);   // U (+ inverse on warp 0)
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
            const uint32_t a0 = tf32r(E[ks][0]), a1 = tf32r(E[ks][2]), a2 = tf32r(E[ks][1]), a3 = tf32r(E[ks][3]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float* pb = Bt + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(X2[nt], a0, a1, a2, a3, __float_as_uint(pb[0]), __float_as_uint(pb[4]));
                const float* pk = Kt + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(X2[2 + nt], a0, a1, a2, a3, __float_as_uint(pk[0]), __float_as_uint(pk[4]));
            }
        }
        WKV7_PHASE(3);   // scale E/ET, X2
        cp_async_wait<1>();   // sa and the chunk-start state have landed (only the next input tiles may be pending)
        __syncthreads();

        WKV7_PHASE(4);   // barrier (inverse, sa, S0)
        // ---- EV and dV ------------------------------------------------------------------------
        {   // sa arrived as fp32: round it to TF32 once (it is only ever an MMA operand here)
            float4* p = reinterpret_cast<float4*>(SAs + lrow * PT + lseg * 8);
            float4 x0 = p[0], x1 = p[1];
            x0.x = tf32rf(x0.x); x0.y = tf32rf(x0.y); x0.z = tf32rf(x0.z); x0.w = tf32rf(x0.w);
            x1.x = tf32rf(x1.x); x1.y = tf32rf(x1.y); x1.z = tf32rf(x1.z); x1.w = tf32rf(x1.w);
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
                EVs[tt * PK + (i & ~7) + perm8(i & 7)] = tf32rf(EV[nt][e]);
            }
        WKV7_PHASE(5);   // EV chain, dV
        __syncthreads();

        // ---- Gram blocks: warp 0 P1 = EV^T V, 1 P3 = EV^T SA, 2 P2 = dY^T V, 3 P4 = dY^T SA ----
        float P[2][4] = {};
        {
            const float* Am = (warp & 2) ? dYf : EVs;
            const float* Bm = (warp & 1) ? SA : Vf;
            uint32_t areg[8][4];
            load_a_plain<8>(areg, Am, PK, 0, g, t);
            if (warp & 1) gemm_rs<2, 8>(P, areg, Bm, PT, g, t);        // sa: natural order, 64-bit reads
            else gemm_rs_plain<2, 8>(P, areg, Bm, PK, g, t);
        }
        WKV7_PHASE(6);   // barrier + Gram
        // ---- Z1 = ETw [V | SA],  Z2 = S0^T [EV | dY]   (rows = key j) ---------------------------
        float Z1[4][4] = {}, Z2[4][4] = {};
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
                const uint2 bs = lds2(SA + (nt * 8 + g) * PT + ks * 8 + 2 * t);
                mma8(Z1[2 + nt], a0, a1, a2, a3, bs.x, bs.y);
                const float* pe = EVs + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z2[nt], s0a, s1a, s2a, s3a, __float_as_uint(pe[0]), __float_as_uint(pe[4]));
                const float* pd = dYf + (nt * 8 + g) * PK + ks * 8 + t;
                mma8(Z2[2 + nt], s0a, s1a, s2a, s3a, __float_as_uint(pd[0]), __float_as_uint(pd[4]));
            }
        }
        WKV7_PHASE(7);   // Z1, Z2
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
                    const float val = tf32rf(keep ? P[nt][e] : 0.f);
                    pn[u * PU + tt] = val;
                    pt[tt * PU + u] = val;
                }
        }
        __syncthreads();

        // ---- dK' dB' (in Z1) and dA' dR' (in Z2) ------------------------------------------------
        // The scaled vectors enter these last small products unrounded (hi + lo TF32 parts, two MMAs):
        // their rounding error is what the decay gradient's running sum would otherwise amplify.
        uint32_t atreg[2][4], rtreg[2][4], btreg[2][4], ktreg[2][4];
        uint32_t atlo[2][4], rtlo[2][4], btlo[2][4], ktlo[2][4];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            float2 wp2 = make_float2(1.f, 1.f);
            if (ks > 0 || t > 0) wp2 = *reinterpret_cast<const float2*>(Wt + (ks * 8 + 2 * t - 1) * PK + row0 + 2 * g);
#pragma unroll
            for (int uh = 0; uh < 2; ++uh) {      // fragment slots e = 2*uh (row g) and 2*uh+1 (row g+8) = real channels 2g, 2g+1
                const int u = ks * 8 + 2 * t + uh, jr = row0 + 2 * g;
                const float2 wu2 = *reinterpret_cast<const float2*>(Wt + u * PK + jr);
                const float2 iw2 = make_float2(frcp(wu2.x), frcp(wu2.y));
                const float2 a2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(A + u * RP + jr));
                const float2 r2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(R + u * RP + jr));
                const float2 b2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(Bv + u * RP + jr));
                const float2 k2 = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(K + u * RP + jr));
                const float xa[2] = {a2.x * wp2.x, a2.y * wp2.y}, xr[2] = {r2.x * wu2.x, r2.y * wu2.y};
                const float xb[2] = {b2.x * iw2.x, b2.y * iw2.y}, xk[2] = {k2.x * iw2.x, k2.y * iw2.y};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int e = 2 * uh + h;
                    atreg[ks][e] = tf32(xa[h]); atlo[ks][e] = tf32r(xa[h] - __uint_as_float(atreg[ks][e]));
                    rtreg[ks][e] = tf32(xr[h]); rtlo[ks][e] = tf32r(xr[h] - __uint_as_float(rtreg[ks][e]));
                    btreg[ks][e] = tf32(xb[h]); btlo[ks][e] = tf32r(xb[h] - __uint_as_float(btreg[ks][e]));
                    ktreg[ks][e] = tf32(xk[h]); ktlo[ks][e] = tf32r(xk[h] - __uint_as_float(ktreg[ks][e]));
                }
                wp2 = wu2;
            }
        }
        WKV7_PHASE(8);   // barrier + hi/lo loaders
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

        WKV7_PHASE(9);   // P products
        // ---- E and ET updates ------------------------------------------------------------------
        gemm_rs_kperm<8, 2>(E, evreg, At, PK, g, t);         // E += EV A~   (B[k=t][n=j] = a~_t[j])
        gemm_rs_kperm<8, 2>(E, dyreg, Rt, PK, g, t);         //    + dY R~
        gemm_rs_kperm<8, 2>(ET, atreg, EVs, PK, g, t);       // ET += A~^T EV^T (B[k=t][n=i] = e_t[i])
        gemm_rs_kperm<8, 2>(ET, rtreg, dYf, PK, g, t);       //     + R~^T dY^T

        WKV7_PHASE(10);  // E, ET updates
        // ---- per-token gradients, rows j = row0+g (+8), columns = tokens --------------------------
        float A0[2] = {0.f, 0.f};                            // sum_i E_start[i,j] S0[i,j]
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
        __syncthreads();      // every warp is done with sa and the staged state
        if (c > 0) issue_state(c - 1); else cp_async_commit();
        WKV7_PHASE(11);  // A0, barrier, state prefetch
        float cterm[2][4], ada[2][4], sgd[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int q = 0; q < 2; ++q) {         // token tt, both rows of the thread: real channels jr, jr+1
                const int tt = nt * 8 + 2 * t + q, jr = row0 + 2 * g;
                const float2 wt = *reinterpret_cast<const float2*>(Wt + tt * PK + jr);
                float2 wprev = make_float2(1.f, 1.f);
                if (tt > 0) wprev = *reinterpret_cast<const float2*>(Wt + (tt - 1) * PK + jr);
                const float2 rr = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(R + tt * RP + jr));
                const float2 aa = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(A + tt * RP + jr));
                const float2 bq = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(Bv + tt * RP + jr));
                const float2 kq = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(K + tt * RP + jr));
                const float2 wr = bf16x2_to_f2(*reinterpret_cast<const uint32_t*>(Wr + tt * RP + jr));
                const float wtv[2] = {wt.x, wt.y}, wpv[2] = {wprev.x, wprev.y};
                const float rv[2] = {rr.x, rr.y}, av[2] = {aa.x, aa.y}, bv2[2] = {bq.x, bq.y}, kv[2] = {kq.x, kq.y}, wv[2] = {wr.x, wr.y};
                float dk[2], db[2], da[2], dr[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int e = 2 * h + q;
                    const float iw = frcp(wtv[h]);
                    dk[h] = Z1[nt][e] * iw; db[h] = Z1[2 + nt][e] * iw;
                    da[h] = Z2[nt][e] * wpv[h]; dr[h] = Z2[2 + nt][e] * wtv[h];
                    ada[nt][e] = av[h] * da[h];
                    cterm[nt][e] = rv[h] * dr[h] + ada[nt][e] - bv2[h] * db[h] - kv[h] * dk[h];
                    const float sg = frcp(1.f + fexp(-wv[h]));
                    sgd[nt][e] = kWScale * sg * (1.f - sg);
                }
                const i64 o = tok0 + (i64)(c * L + tt) * C + jr;
                *reinterpret_cast<uint32_t*>(dk_ + o) = f2_to_bf16x2(dk[0], dk[1]);
                *reinterpret_cast<uint32_t*>(db_ + o) = f2_to_bf16x2(db[0], db[1]);
                *reinterpret_cast<uint32_t*>(da_ + o) = f2_to_bf16x2(da[0], da[1]);
                *reinterpret_cast<uint32_t*>(dr_ + o) = f2_to_bf16x2(dr[0], dr[1]);
            }
        WKV7_PHASE(12);  // dk db da dr
        // exclusive prefix of cterm along the 16 tokens of each row: lanes t = 0..3 of a quad hold
        // tokens (2t, 2t+1) of tile 0 and (8+2t, 8+2t+1) of tile 1
        float G[2][4];
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
                G[h2][q] = (A0[h2] - pre[q] - ada[nt][e]) * sgd[nt][e];
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int tt = (q >> 1) * 8 + 2 * t + (q & 1);
            *reinterpret_cast<uint32_t*>(dw_ + tok0 + (i64)(c * L + tt) * C + row0 + 2 * g) = f2_to_bf16x2(G[0][q], G[1][q]);
        }
        WKV7_PHASE(13);  // dw
    }

    if (ds0_ != nullptr) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {   // logical columns of tiles 2m, 2m+1 = real columns 16m + 4t .. 16m + 4t + 3
            *reinterpret_cast<float4*>(ds0_ + sbase + (row0 + g) * N + 16 * m + 4 * t) =
                make_float4(E[2 * m][0], E[2 * m + 1][0], E[2 * m][1], E[2 * m + 1][1]);
            *reinterpret_cast<float4*>(ds0_ + sbase + (row0 + g + 8) * N + 16 * m + 4 * t) =
                make_float4(E[2 * m][2], E[2 * m + 1][2], E[2 * m][3], E[2 * m + 1][3]);
        }
    }
}

WKV7_PHASE_READER(rwkvb200_phase_clocks_chunked_bwd)

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
