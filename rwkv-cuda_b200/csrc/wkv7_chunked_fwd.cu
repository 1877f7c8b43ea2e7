// RWKV-7 forward, head size 64, bf16 activations: chunked tensor-core kernel.
//
// One CTA (4 warps) per (batch, head).  The 64x64 fp32 state lives in registers as MMA
// accumulator tiles, warp w holding rows 16w..16w+15, and never leaves them: it is the A operand
// of the next chunk's products as it stands (see the k-permutation note in wkv7_chunked.cuh).
// Per chunk of 16 tokens:
//   load   six [16 x 64] bf16 input tiles by cp.async into a 2-stage ring (the next chunk's
//          tiles are in flight while this one is computed)
//   prep   per-channel decays, their cumulative products, the six scaled operand arrays
//   small  U_ab, U_ak, U_br, U_kr (one per warp, 16 MMAs each) and T = (I - U_ab)^-1 in fp32
//   chain  X = S [A~|R~]; SA = (X_a + V U_ak) T; Y = X_r + SA U_br + V U_kr; S = S We + SA B^ + V K^
//   store  y (bf16) and sa (fp32) through a shared-memory transpose as full 128/256-byte rows,
//          and the chunk-start state straight from the accumulator registers.
// Saved for the backward: s[b,h,c] = state at the START of chunk c (row-major [value][key]),
// sa[b,t,h,:] = S_{t-1} a_t.
#include "wkv7_chunked.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7c {

// shared memory map (floats unless noted)
struct FwdSmem {
    static constexpr int kRaw = 0;                                   // bf16 [2][6][L*N]
    static constexpr int kRawBytes = 2 * 6 * L * N * 2;
    static constexpr int kAt = kRawBytes / 4;                        // a~ token-major [L][PT]; reused as y staging
    static constexpr int kRt = kAt + L * PT;                         // r~;                     reused as sa staging
    static constexpr int kBt = kRt + L * PT;                         // b~ token-major [L][PK], channels permuted
    static constexpr int kKt = kBt + L * PK;                         // k~
    static constexpr int kVf = kKt + L * PK;                         // v as fp32, token-major [L][PK]
    static constexpr int kUab = kVf + L * PK;                        // [s][t], fp32
    static constexpr int kUak = kUab + L * PU;                       // [t][s], tf32
    static constexpr int kUbr = kUak + L * PU;
    static constexpr int kUkr = kUbr + L * PU;
    static constexpr int kTt = kUkr + L * PU;
    static constexpr int kWe = kTt + L * PU;                         // [N]
    static constexpr int kHalf = kWe + N;                            // [2][N] half-chunk log-decay sums
    static constexpr int kEnd = kHalf + 2 * N;
    static constexpr int kBytes = kEnd * 4;
};
static_assert(L * PS <= L * PT, "staging must fit in the arrays it reuses");

__global__ void __launch_bounds__(NT, 4)
wkv7c_forward_kernel(int T, int H, const float* __restrict__ s0_, const bf16* __restrict__ r_,
                     const bf16* __restrict__ w_, const bf16* __restrict__ k_, const bf16* __restrict__ v_,
                     const bf16* __restrict__ a_, const bf16* __restrict__ b_, bf16* __restrict__ y_,
                     float* __restrict__ sT_, float* __restrict__ ck_, float* __restrict__ sa_) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* sm = reinterpret_cast<float*>(smem_raw);
    bf16* raw = reinterpret_cast<bf16*>(smem_raw);
    float *At = sm + FwdSmem::kAt, *Rt = sm + FwdSmem::kRt, *Bt = sm + FwdSmem::kBt, *Kt = sm + FwdSmem::kKt;
    float* Vf = sm + FwdSmem::kVf;
    float *Uab = sm + FwdSmem::kUab, *Uak = sm + FwdSmem::kUak, *Ubr = sm + FwdSmem::kUbr, *Ukr = sm + FwdSmem::kUkr;
    float *Tt = sm + FwdSmem::kTt, *We = sm + FwdSmem::kWe, *Hs = sm + FwdSmem::kHalf;
    float *ystage = At, *sastage = Rt;

    const int hh = blockIdx.x, bb = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row0 = warp * 16;
    const int C = H * N;
    const i64 tok0 = (i64)bb * T * C + hh * N;
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const int nchunks = T / L;
    float* ck = ck_ ? ck_ + (i64)(bb * H + hh) * nchunks * N * N : nullptr;
    const bf16* src[6] = {r_, w_, k_, v_, a_, b_};

    // state tiles: S[nt] = rows row0+g / row0+g+8, columns 8nt+2t, 8nt+2t+1
    float S[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        float2 lo = make_float2(0.f, 0.f), hi = lo;
        if (s0_ != nullptr) {
            lo = *reinterpret_cast<const float2*>(s0_ + sbase + (row0 + g) * N + nt * 8 + 2 * t);
            hi = *reinterpret_cast<const float2*>(s0_ + sbase + (row0 + g + 8) * N + nt * 8 + 2 * t);
        }
        S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
    }

    const int lrow = tid >> 3, lseg = tid & 7;  // cp.async / store mapping: token row, 8-channel segment
    auto issue_loads = [&](int c, int stage) {
        const i64 off = tok0 + (i64)(c * L + lrow) * C + lseg * 8;
#pragma unroll
        for (int x = 0; x < 6; ++x) cp_async16(raw + ((stage * 6 + x) * L + lrow) * N + lseg * 8, src[x] + off);
        cp_async_commit();
    };
    issue_loads(0, 0);

    for (int c = 0; c < nchunks; ++c) {
        const int stage = c & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (c + 1 < nchunks) issue_loads(c + 1, stage ^ 1);
        const bf16* R = raw + (stage * 6 + 0) * L * N;
        const bf16* Wr = raw + (stage * 6 + 1) * L * N;
        const bf16* K = raw + (stage * 6 + 2) * L * N;
        const bf16* V = raw + (stage * 6 + 3) * L * N;
        const bf16* A = raw + (stage * 6 + 4) * L * N;
        const bf16* Bv = raw + (stage * 6 + 5) * L * N;

        // ---- prep: thread = (channel j, half of the chunk) ------------------------------------
        {
            const int j = tid & 63, hf = tid >> 6, t0 = hf * 8;
            float cs[8];
            float run = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float x = to_f(Wr[(t0 + q) * N + j]);
                run = fmaf(kWScale2, frcp(1.f + fexp(-x)), run);  // log decay, cumulative within the half
                cs[q] = run;
            }
            Hs[hf * N + j] = run;
            __syncthreads();
            const float base = hf ? Hs[j] : 0.f;
            const float lam_e = Hs[j] + Hs[N + j];
            if (hf == 0) We[j] = fex2(lam_e);
            float wprev = hf ? fex2(base) : 1.f;
            const int jp = (j & ~7) + perm8(j & 7);
            // loads of a batch of four tokens before its stores (tiles and operand arrays share one
            // shared-memory block: the compiler keeps a load behind every earlier store)
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                float xa[4], xr[4], xb[4], xk[4], xv[4], wt[4], iw[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int tt = t0 + 4 * hb + q;
                    xa[q] = to_f(A[tt * N + j]); xr[q] = to_f(R[tt * N + j]); xb[q] = to_f(Bv[tt * N + j]);
                    xk[q] = to_f(K[tt * N + j]); xv[q] = to_f(V[tt * N + j]);
                    const float lam = base + cs[4 * hb + q];
                    wt[q] = fex2(lam); iw[q] = fex2(-lam);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int tt = t0 + 4 * hb + q;
                    At[tt * PT + j] = tf32f(xa[q] * wprev);
                    Rt[tt * PT + j] = tf32f(xr[q] * wt[q]);
                    Bt[tt * PK + jp] = tf32f(xb[q] * iw[q]);
                    Kt[tt * PK + jp] = tf32f(xk[q] * iw[q]);
                    Vf[tt * PK + j] = xv[q];
                    wprev = wt[q];
                }
            }
        }
        __syncthreads();

        // ---- small products: warp 0 U_ab (+T), 1 U_ak, 2 U_br, 3 U_kr -------------------------
        {
            const float* Am = (warp & 1) ? Kt : Bt;
            const float* Bm = (warp & 2) ? Rt : At;
            uint32_t areg[8][4];
            load_a_plain<8>(areg, Am, PK, 0, g, t);
            float U[2][4] = {};
            gemm_rs<2, 8>(U, areg, Bm, PT, g, t);
            float* dst = warp == 0 ? Uab : warp == 1 ? Uak : warp == 2 ? Ubr : Ukr;
            const bool strict = warp < 2;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int s = g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                    const bool keep = strict ? (s < tt) : (s <= tt);
                    const float val = keep ? U[nt][e] : 0.f;
                    if (warp == 0) dst[s * PU + tt] = val;
                    else dst[tt * PU + s] = tf32f(val);
                }
            if (warp == 0) {
                __syncwarp();
                tri_inverse(Uab, Tt, lane);
            }
        }

        // ---- X = S [A~ | R~]  (needs only the prep arrays) --------------------------------------
        float X[4][4] = {};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a0 = tf32(S[ks][0]), a1 = tf32(S[ks][2]), a2 = tf32(S[ks][1]), a3 = tf32(S[ks][3]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const uint2 ba = lds2(At + (nt * 8 + g) * PT + ks * 8 + 2 * t);
                mma8(X[nt], a0, a1, a2, a3, ba.x, ba.y);
                const uint2 br = lds2(Rt + (nt * 8 + g) * PT + ks * 8 + 2 * t);
                mma8(X[2 + nt], a0, a1, a2, a3, br.x, br.y);
            }
        }
        __syncthreads();

        // ---- the state chain -------------------------------------------------------------------
        uint32_t vreg[2][4], xreg[2][4], sareg[2][4];
        load_a_kmaj<2>(vreg, Vf, PK, row0, g, t);
        gemm_rs<2, 2>(X, vreg, Uak, PU, g, t);           // X_a += V U_ak
        acc_to_a<2>(xreg, X);
        float SA[2][4] = {};
        gemm_rs<2, 2>(SA, xreg, Tt, PU, g, t);           // SA = X_a T
        acc_to_a<2>(sareg, SA);
        gemm_rs<2, 2>(X + 2, sareg, Ubr, PU, g, t);      // Y = X_r + SA U_br + V U_kr
        gemm_rs<2, 2>(X + 2, vreg, Ukr, PU, g, t);

        if (ck != nullptr) {  // state at the start of this chunk
            float* dst = ck + (i64)c * N * N;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                *reinterpret_cast<float2*>(dst + (row0 + g) * N + nt * 8 + 2 * t) = make_float2(S[nt][0], S[nt][1]);
                *reinterpret_cast<float2*>(dst + (row0 + g + 8) * N + nt * 8 + 2 * t) = make_float2(S[nt][2], S[nt][3]);
            }
        }
        gemm_rs_kperm<8, 2>(S, sareg, Bt, PK, g, t);      // S = (S + SA B~ + V K~) diag(We)
        gemm_rs_kperm<8, 2>(S, vreg, Kt, PK, g, t);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float2 we = *reinterpret_cast<const float2*>(We + nt * 8 + 2 * t);
            S[nt][0] *= we.x; S[nt][1] *= we.y; S[nt][2] *= we.x; S[nt][3] *= we.y;
        }

        // ---- y and sa: transpose through shared memory, then full-row stores -------------------
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = row0 + g + ((e & 2) ? 8 : 0), tt = nt * 8 + 2 * t + (e & 1);
                ystage[tt * PS + i] = X[2 + nt][e];
                sastage[tt * PS + i] = SA[nt][e];
            }
        __syncthreads();
        {
            const i64 off = tok0 + (i64)(c * L + lrow) * C + lseg * 8;
            const float4 y0 = *reinterpret_cast<const float4*>(ystage + lrow * PS + lseg * 8);
            const float4 y1 = *reinterpret_cast<const float4*>(ystage + lrow * PS + lseg * 8 + 4);
            __nv_bfloat162 p0 = __floats2bfloat162_rn(y0.x, y0.y), p1 = __floats2bfloat162_rn(y0.z, y0.w);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(y1.x, y1.y), p3 = __floats2bfloat162_rn(y1.z, y1.w);
            uint4 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
            pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
            *reinterpret_cast<uint4*>(y_ + off) = pk;
            if (sa_ != nullptr) {
                float4* d = reinterpret_cast<float4*>(sa_ + off);
                d[0] = *reinterpret_cast<const float4*>(sastage + lrow * PS + lseg * 8);
                d[1] = *reinterpret_cast<const float4*>(sastage + lrow * PS + lseg * 8 + 4);
            }
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

}  // namespace v7c

int wkv7_chunked_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k,
                         const void* v, const void* a, const void* b, void* y, float* sT, float* s, float* sa,
                         cudaStream_t st) {
    using namespace v7c;
    static_assert(FwdSmem::kBytes <= 55 * 1024 + 768, "forward shared memory must allow 4 CTAs per SM");
    cudaError_t e = cudaFuncSetAttribute(wkv7c_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem::kBytes);
    RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "wkv7_forward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    dim3 grid(H, B);
    wkv7c_forward_kernel<<<grid, NT, FwdSmem::kBytes, st>>>(T, H, s0, (const bf16*)r, (const bf16*)w, (const bf16*)k,
                                                            (const bf16*)v, (const bf16*)a, (const bf16*)b, (bf16*)y,
                                                            sT, s, sa);
    return check_launch("wkv7_forward(chunked)");
}

}  // namespace rwkvb200
