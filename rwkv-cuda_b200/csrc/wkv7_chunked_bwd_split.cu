// RWKV-7 backward, head size 64, bf16 activations: the chunked mma.sync kernel of
// wkv7_chunked_bwd.cu as a producer/consumer pair, for launches that put at most one (batch, head)
// unit on an SM (B*H <= number of SMs: strong scaling over GPUs at a small batch per GPU).
//
// With one CTA per SM the time of the backward is the length of one unit's chain of chunks, and in
// wkv7_chunked_bwd.cu a third of every chunk is work that does not depend on the carried state
// gradients: operand preparation, the four U matrices and the 16x16 inverse.  Here a second group
// of four warps (the producers) does exactly that work one chunk ahead, into a second set of operand
// arrays, while the first four warps (the consumers, who own E and ET) run the rest of the chunk.
// The producers also take the consumers' last step off their hands: the per-token epilogue (dr, dw,
// dk, da, db from Z1, Z2 and A0, handed over through shared memory), one chunk behind.
// One CTA-wide barrier per chunk hands the finished set over and returns the other; inside a group
// the barriers are named barriers of 128 threads.  Input tiles go through a ring of three stages
// (read by the consumers' epilogue, read by the producers, in flight).  Same arithmetic, same
// fragment layouts and results as wkv7_chunked_bwd.cu; 201 KB of shared memory, one CTA per SM.
#include "wkv7_chunked.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7s {

using namespace v7c;

constexpr int PS0 = 68;            // pitch of the staged 64x64 state
constexpr int NTS = 2 * NT;        // 8 warps: consumers 0-3, producers 4-7
constexpr int kSetFloats = 7 * L * PK + 5 * L * PU + N;   // At Rt Bt Kt Vf dYf Wt | Uab Uak Ubr Ukr T | We

struct SSmem {
    static constexpr int kRawBytes = 3 * 7 * L * RP * 2;             // bf16 [3][7][L][RP]: r w k v a b dy
    static constexpr int kSets = kRawBytes / 4;                      // two operand sets
    static constexpr int kSa = kSets + 2 * kSetFloats;               // fp32 [L][PT]
    static constexpr int kS0 = kSa + L * PT;                         // fp32 [N][PS0]
    static constexpr int kEv = kS0 + N * PS0;                        // EV [t][i]
    static constexpr int kP = kEv + L * PK;                          // P1..P4 natural, then transposed
    static constexpr int kHalf = kP + 8 * L * PU;
    static constexpr int kZb = kHalf + 2 * N;                        // [2][9][NT] float4: Z1, Z2 and A0 of a finished chunk
    static constexpr int kEnd = kZb + 2 * 9 * NT * 4;
    static constexpr int kBytes = kEnd * 4;
};
static_assert(SSmem::kBytes <= 227 * 1024, "shared memory of the producer/consumer backward");

__device__ __forceinline__ void store_bf16(bf16* p, float x) { *p = __float2bfloat16_rn(x); }

__global__ void __launch_bounds__(NTS, 1)
wkv7s_backward_kernel(int T, int H, const bf16* __restrict__ r_, const bf16* __restrict__ w_,
                      const bf16* __restrict__ k_, const bf16* __restrict__ v_, const bf16* __restrict__ a_,
                      const bf16* __restrict__ b_, const bf16* __restrict__ dy_, const float* __restrict__ dsT_,
                      const float* __restrict__ ck_, const float* __restrict__ sa_, float* __restrict__ ds0_,
                      bf16* __restrict__ dr_, bf16* __restrict__ dw_, bf16* __restrict__ dk_, bf16* __restrict__ dv_,
                      bf16* __restrict__ da_, bf16* __restrict__ db_) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* sm = reinterpret_cast<float*>(smem_raw);
    bf16* raw = reinterpret_cast<bf16*>(smem_raw);
    float *SAs = sm + SSmem::kSa, *S0s = sm + SSmem::kS0, *EVs = sm + SSmem::kEv;
    float *Pn = sm + SSmem::kP, *Ptr = Pn + 4 * L * PU;   // natural / transposed, index 0..3 = P1..P4
    float* Hs = sm + SSmem::kHalf;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const bool producer = threadIdx.x >= NT;
    // group-local indices: each group of four warps is laid out like the CTA of wkv7_chunked_bwd.cu
    const int tid = threadIdx.x & (NT - 1), warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = warp * 16;
    const int C = H * N;
    const i64 tok0 = (i64)bb * T * C + hh * N;
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const int nchunks = T / L;
    const float* ck = ck_ + (i64)(bb * H + hh) * nchunks * N * N;
    const bf16* src[7] = {r_, w_, k_, v_, a_, b_, dy_};
    auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(producer ? 2 : 1) : "memory"); };

    const int lrow = tid >> 3, lseg = tid & 7;
    auto issue_raw = [&](int c) {   // producers
        const int stage = c % 3;
        const i64 off = tok0 + (i64)(c * L + lrow) * C + lseg * 8;
#pragma unroll
        for (int x = 0; x < 7; ++x) cp_async16(raw + ((stage * 7 + x) * L + lrow) * RP + lseg * 8, src[x] + off);
        cp_async_commit();
    };
    // sa (16 x 64 fp32) and the chunk-start state (64 x 64 fp32) are single-buffered (consumers)
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

    // E[nt]: rows i = row0+g / +8, cols j = 8nt+2t (+1).  ET[nt]: rows j = row0+g / +8, cols i = 8nt+2t (+1).
    // (consumers only; the producers leave them untouched)
    float E[8][4], ET[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = row0 + g + ((e & 2) ? 8 : 0), col = nt * 8 + 2 * t + (e & 1);
            E[nt][e] = (dsT_ && !producer) ? dsT_[sbase + row * N + key_real(col)] : 0.f;
            ET[nt][e] = (dsT_ && !producer) ? dsT_[sbase + col * N + key_real(row)] : 0.f;
        }

    // operand preparation, the U matrices and T = (I - U_ab)^-1 of chunk c into its operand set
    auto produce = [&](int c) {
        const int stage = c % 3;
        float* set = sm + SSmem::kSets + (c & 1) * kSetFloats;
        float *At = set, *Rt = At + L * PK, *Bt = Rt + L * PK, *Kt = Bt + L * PK, *Vf = Kt + L * PK, *dYf = Vf + L * PK;
        float* Wt = dYf + L * PK;
        float *Uab = Wt + L * PK, *Tn = Uab + 4 * L * PU, *We = Uab + 5 * L * PU;
        const bf16* R = raw + (stage * 7 + 0) * L * RP;
        const bf16* Wr = raw + (stage * 7 + 1) * L * RP;
        const bf16* K = raw + (stage * 7 + 2) * L * RP;
        const bf16* V = raw + (stage * 7 + 3) * L * RP;
        const bf16* A = raw + (stage * 7 + 4) * L * RP;
        const bf16* Bv = raw + (stage * 7 + 5) * L * RP;
        const bf16* DY = raw + (stage * 7 + 6) * L * RP;
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
                group_sync();
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
            group_sync();
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
    };

    // per-token gradients of a finished chunk ce from its Z1 (dK', dB'), Z2 (dA', dR') and A0: rows = real
    // key channels row0+2g (+1), columns = tokens.  Run by the producers, one chunk behind the consumers.
    auto epilogue = [&](int ce) {
        const int stage = ce % 3;
        const float* Wt = sm + SSmem::kSets + (ce & 1) * kSetFloats + 6 * L * PK;
        const bf16* R = raw + (stage * 7 + 0) * L * RP;
        const bf16* Wr = raw + (stage * 7 + 1) * L * RP;
        const bf16* K = raw + (stage * 7 + 2) * L * RP;
        const bf16* A = raw + (stage * 7 + 4) * L * RP;
        const bf16* Bv = raw + (stage * 7 + 5) * L * RP;
        float Z1[4][4], Z2[4][4], A0[2];
        {
            const float4* zb = reinterpret_cast<const float4*>(sm + SSmem::kZb) + (ce & 1) * 9 * NT + tid;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 x = zb[q * NT], y = zb[(4 + q) * NT];
                Z1[q][0] = x.x; Z1[q][1] = x.y; Z1[q][2] = x.z; Z1[q][3] = x.w;
                Z2[q][0] = y.x; Z2[q][1] = y.y; Z2[q][2] = y.z; Z2[q][3] = y.w;
            }
            const float4 a0 = zb[8 * NT];
            A0[0] = a0.x; A0[1] = a0.y;
        }
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
                const i64 o = tok0 + (i64)(ce * L + tt) * C + jr;
                *reinterpret_cast<uint32_t*>(dk_ + o) = f2_to_bf16x2(dk[0], dk[1]);
                *reinterpret_cast<uint32_t*>(db_ + o) = f2_to_bf16x2(db[0], db[1]);
                *reinterpret_cast<uint32_t*>(da_ + o) = f2_to_bf16x2(da[0], da[1]);
                *reinterpret_cast<uint32_t*>(dr_ + o) = f2_to_bf16x2(dr[0], dr[1]);
            }
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
            *reinterpret_cast<uint32_t*>(dw_ + tok0 + (i64)(ce * L + tt) * C + row0 + 2 * g) = f2_to_bf16x2(G[0][q], G[1][q]);
        }
    };

    if (producer) {
        issue_raw(nchunks - 1);
        if (nchunks > 1) issue_raw(nchunks - 2); else cp_async_commit();
        cp_async_wait<1>();
        group_sync();
        produce(nchunks - 1);
    } else {
        issue_state(nchunks - 1);
    }
    __syncthreads();

    for (int c = nchunks - 1; c >= 0; --c) {
        if (producer) {
            if (c + 1 < nchunks) {
                epilogue(c + 1);   // needs the tiles and W_t of chunk c+1, which the steps below overwrite
                group_sync();
            }
            if (c > 0) {
                if (c > 1) issue_raw(c - 2); else cp_async_commit();   // its stage held chunk c+1, which nobody reads any more
                cp_async_wait<1>();                                      // the tiles of chunk c-1 have landed
                group_sync();
                produce(c - 1);
            }
        } else {
            const int stage = c % 3;
            float* set = sm + SSmem::kSets + (c & 1) * kSetFloats;
            float *At = set, *Rt = At + L * PK, *Bt = Rt + L * PK, *Kt = Bt + L * PK, *Vf = Kt + L * PK, *dYf = Vf + L * PK;
            float* Wt = dYf + L * PK;
            float *Uab = Wt + L * PK, *Uak = Uab + L * PU, *Ubr = Uak + L * PU, *Ukr = Ubr + L * PU, *Tn = Ukr + L * PU;
            float* We = Uab + 5 * L * PU;
            const bf16* R = raw + (stage * 7 + 0) * L * RP;
            const bf16* K = raw + (stage * 7 + 2) * L * RP;
            const bf16* A = raw + (stage * 7 + 4) * L * RP;
            const bf16* Bv = raw + (stage * 7 + 5) * L * RP;
            const float* SA = SAs;
            const float* S0 = S0s;
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
            cp_async_wait<0>();   // sa and the chunk-start state have landed
            group_sync();
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
            group_sync();

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
            group_sync();

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
            group_sync();      // every warp is done with sa and the staged state
            if (c > 0) issue_state(c - 1);
            {   // Z1, Z2 and A0 go to the producers, who turn them into dr, dw, dk, da, db while the next chunk runs
                float4* zb = reinterpret_cast<float4*>(sm + SSmem::kZb) + (c & 1) * 9 * NT + tid;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    zb[q * NT] = make_float4(Z1[q][0], Z1[q][1], Z1[q][2], Z1[q][3]);
                    zb[(4 + q) * NT] = make_float4(Z2[q][0], Z2[q][1], Z2[q][2], Z2[q][3]);
                }
                zb[8 * NT] = make_float4(A0[0], A0[1], 0.f, 0.f);
            }
        }
        __syncthreads();   // hand-over: the set of chunk c-1 is complete, the set and the tiles of chunk c are free
    }

    if (producer) epilogue(0);
    if (!producer && ds0_ != nullptr) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {   // logical columns of tiles 2m, 2m+1 = real columns 16m + 4t .. 16m + 4t + 3
            *reinterpret_cast<float4*>(ds0_ + sbase + (row0 + g) * N + 16 * m + 4 * t) =
                make_float4(E[2 * m][0], E[2 * m + 1][0], E[2 * m][1], E[2 * m + 1][1]);
            *reinterpret_cast<float4*>(ds0_ + sbase + (row0 + g + 8) * N + 16 * m + 4 * t) =
                make_float4(E[2 * m][2], E[2 * m + 1][2], E[2 * m][3], E[2 * m + 1][3]);
        }
    }
}

}  // namespace v7s

int wkv7_split_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v,
                        const void* a, const void* b, const void* dy, const float* dsT, const float* s,
                        const float* sa, float* ds0, void* dr, void* dw, void* dk, void* dv, void* da, void* db,
                        cudaStream_t st) {
    using namespace v7s;
    cudaError_t e = cudaFuncSetAttribute(wkv7s_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SSmem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_backward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7s_backward_kernel<<<grid, NTS, SSmem::kBytes, st>>>(
        T, H, (const bf16*)r, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b,
        (const bf16*)dy, dsT, s, sa, ds0, (bf16*)dr, (bf16*)dw, (bf16*)dk, (bf16*)dv, (bf16*)da, (bf16*)db);
    return check_launch("wkv7_backward(producer/consumer)");
}

}  // namespace rwkvb200
