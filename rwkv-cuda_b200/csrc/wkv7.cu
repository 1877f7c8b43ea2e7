// RWKV-7 generalised delta rule with soft-clamped decay: general-shape kernels
// (any head size N <= 128, fp32 or bf16 activations, fp32 state).
//
// Operator (rwkv7_fast_fused/rwkv7_cuda_benchmark_state_passing.py:46-68 of the reference
// project), per (b,h), S indexed [value i][key j]:
//   d_t = exp(-e^{-1/2} sigmoid(w_raw_t))
//   sa  = S a_t ;  S <- S diag(d_t) + sa b_t^T + v_t k_t^T ;  y_t = S r_t
// with optional initial state s0, final state sT, and in the backward dsT in / ds0 out.
//
// One CTA per (batch, head); thread i owns row i of S in registers.  Per-token vectors go
// through a double-buffered shared-memory stage (one barrier per token in the forward, two in
// the backward) and the next token's elements are fetched while the current one is computed.
// The forward saves sa_t and a transposed copy of S every `chunk_len` tokens; the backward
// walks time in reverse, reloads S at chunk ends and in between undoes the update
// (S_prev = (S - v k^T - sa b^T) / d, safe because the soft clamp keeps d >= 0.545).
// These kernels serve every shape; the N = 64 bf16 case has a tensor-core path of its own.
#include "common.cuh"

namespace rwkvb200 {
namespace {

constexpr float kWScale = -0.6065306597126334f;  // -exp(-1/2)

template <int NMAX>
struct __align__(16) Stage {
    float a[2][NMAX];
};

constexpr int kAhead = 8;   // tokens between the L1 request for a token's rows and their use

template <typename E, int NMAX>
__global__ void __launch_bounds__(NMAX) wkv7_forward_kernel(int T, int H, int N, int chunk, const float* __restrict__ s0_,
                                                           const E* __restrict__ r_, const E* __restrict__ w_,
                                                           const E* __restrict__ k_, const E* __restrict__ v_,
                                                           const E* __restrict__ a_, const E* __restrict__ b_,
                                                           E* __restrict__ y_, float* __restrict__ sT_,
                                                           float* __restrict__ ck_, float* __restrict__ sa_) {
    const int bb = blockIdx.y, hh = blockIdx.x, i = threadIdx.x;
    const bool live = i < N;
    __shared__ Stage<NMAX> rs, ds, ks, as, bs;
    const i64 sbase = ((i64)(bb * H + hh) * N + i) * N;
    float S[NMAX];
#pragma unroll
    for (int j = 0; j < NMAX; ++j) S[j] = (live && j < N && s0_ != nullptr) ? s0_[sbase + j] : 0.f;

    const int C = H * N;
    const i64 base = (i64)bb * T * C + hh * N + i;
    float* ck = ck_ ? ck_ + (i64)(bb * H + hh) * (T / chunk) * N * N : nullptr;

    // one thread per 128-byte line of a row of N elements asks for the rows of the token kAhead steps on
    const bool line_lead = i == 0 || (reinterpret_cast<uintptr_t>(r_ + base) & 127) < sizeof(E);
    float rn = 0.f, wn = 0.f, kn = 0.f, vn = 0.f, an = 0.f, bn = 0.f;
    if (live) {
        rn = to_f(r_[base]); wn = to_f(w_[base]); kn = to_f(k_[base]);
        vn = to_f(v_[base]); an = to_f(a_[base]); bn = to_f(b_[base]);
    }
    for (int t = 0; t < T; ++t) {
        const int p = t & 1;
        rs.a[p][i] = rn;
        ds.a[p][i] = live ? __expf(kWScale * __fdividef(1.f, 1.f + __expf(-wn))) : 0.f;   // hardware exp2 / reciprocal: as the reference's build does
        ks.a[p][i] = kn; as.a[p][i] = an; bs.a[p][i] = bn;
        const float v = vn;
        __syncthreads();
        if (t + 1 < T && live) {
            const i64 o = base + (i64)(t + 1) * C;
            rn = to_f(r_[o]); wn = to_f(w_[o]); kn = to_f(k_[o]);
            vn = to_f(v_[o]); an = to_f(a_[o]); bn = to_f(b_[o]);
        }
        if (t + kAhead < T && live && line_lead) {   // the rows of a later token into L1: the loads above then find them there
            const i64 o = base + (i64)(t + kAhead) * C;
            prefetch_l1(r_ + o); prefetch_l1(w_ + o); prefetch_l1(k_ + o);
            prefetch_l1(v_ + o); prefetch_l1(a_ + o); prefetch_l1(b_ + o);
        }
        float sa;
        {   // four partial sums: one chain of NMAX dependent multiply-adds would be bound by their latency
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int j = 0; j < NMAX; j += 4) {
                const float4 a4 = *reinterpret_cast<const float4*>(&as.a[p][j]);
                s0 = fmaf(S[j], a4.x, s0); s1 = fmaf(S[j + 1], a4.y, s1);
                s2 = fmaf(S[j + 2], a4.z, s2); s3 = fmaf(S[j + 3], a4.w, s3);
            }
            sa = (s0 + s1) + (s2 + s3);
        }
        float y = 0.f;
#pragma unroll
        for (int j = 0; j < NMAX; j += 4) {
            const float4 d4 = *reinterpret_cast<const float4*>(&ds.a[p][j]);
            const float4 b4 = *reinterpret_cast<const float4*>(&bs.a[p][j]);
            const float4 k4 = *reinterpret_cast<const float4*>(&ks.a[p][j]);
            const float4 r4 = *reinterpret_cast<const float4*>(&rs.a[p][j]);
            const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float s = fmaf(S[j + e], dd[e], fmaf(sa, bv[e], kk[e] * v));
                y = fmaf(s, rr[e], y);
                S[j + e] = s;
            }
        }
        if (live) {
            y_[base + (i64)t * C] = from_f<E>(y);
            if (sa_) sa_[base + (i64)t * C] = sa;
            if (ck && (t + 1) % chunk == 0) {
                float* dst = ck + (i64)(t / chunk) * N * N + i;  // transposed: [key j][value i]
#pragma unroll
                for (int j = 0; j < NMAX; ++j)
                    if (j < N) dst[(i64)j * N] = S[j];
            }
        }
    }
    if (sT_ != nullptr && live) {
#pragma unroll
        for (int j = 0; j < NMAX; ++j)
            if (j < N) sT_[sbase + j] = S[j];
    }
}

template <typename E, int NMAX>
__global__ void __launch_bounds__(NMAX) wkv7_backward_kernel(
    int T, int H, int N, int chunk, const E* __restrict__ r_, const E* __restrict__ w_, const E* __restrict__ k_,
    const E* __restrict__ v_, const E* __restrict__ a_, const E* __restrict__ b_, const E* __restrict__ dy_,
    const float* __restrict__ dsT_, const float* __restrict__ ck_, const float* __restrict__ sa_,
    float* __restrict__ ds0_, E* __restrict__ dr_, E* __restrict__ dw_, E* __restrict__ dk_, E* __restrict__ dv_,
    E* __restrict__ da_, E* __restrict__ db_) {
    const int bb = blockIdx.y, hh = blockIdx.x, i = threadIdx.x;
    const bool live = i < N;
    __shared__ Stage<NMAX> rs, ds, ks, vs, as, bs, gs, ss;
    __shared__ __align__(16) float dsb[NMAX];
    const i64 sbase = (i64)(bb * H + hh) * N * N;
    const float* ck = ck_ + (i64)(bb * H + hh) * (T / chunk) * N * N;

    // ST[j] = S[value j][key i];  DT[j] = dS[value j][key i];  DR[j] = dS[value i][key j]
    float ST[NMAX], DT[NMAX], DR[NMAX];
#pragma unroll
    for (int j = 0; j < NMAX; ++j) {
        const bool in = live && j < N && dsT_ != nullptr;
        ST[j] = 0.f;
        DR[j] = in ? dsT_[sbase + (i64)i * N + j] : 0.f;
        DT[j] = in ? dsT_[sbase + (i64)j * N + i] : 0.f;
    }

    const int C = H * N;
    const i64 base = (i64)bb * T * C + hh * N + i;
    const bool line_lead = i == 0 || (reinterpret_cast<uintptr_t>(r_ + base) & 127) < sizeof(E);
    const bool line_lead_sa = i == 0 || (reinterpret_cast<uintptr_t>(sa_ + base) & 127) < sizeof(float);
    float rn = 0.f, wn = 0.f, kn = 0.f, vn = 0.f, an = 0.f, bn = 0.f, gn = 0.f, sn = 0.f;
    if (live) {
        const i64 o = base + (i64)(T - 1) * C;
        rn = to_f(r_[o]); wn = to_f(w_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]);
        an = to_f(a_[o]); bn = to_f(b_[o]); gn = to_f(dy_[o]); sn = sa_[o];
    }
    for (int t = T - 1; t >= 0; --t) {
        const int p = t & 1;
        // hardware exp2 / reciprocal (as the reference's build does); the accurate forms cost the loop below its registers
        const float sig = __fdividef(1.f, 1.f + __expf(-wn));
        const float di = live ? __expf(kWScale * sig) : 1.f;
        const float ri = rn, ki = kn, ai = an, bi = bn, gi = gn;
        rs.a[p][i] = rn; ds.a[p][i] = live ? di : 0.f; ks.a[p][i] = kn; vs.a[p][i] = vn;
        as.a[p][i] = an; bs.a[p][i] = bn; gs.a[p][i] = gn; ss.a[p][i] = sn;
        __syncthreads();
        if ((t + 1) % chunk == 0 && live) {
            const float* src = ck + (i64)(t / chunk) * N * N + (i64)i * N;
#pragma unroll
            for (int j = 0; j < NMAX; ++j)
                if (j < N) ST[j] = src[j];
        }
        float dr;
        {   // four partial sums: one chain of NMAX dependent multiply-adds would be bound by their latency
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int j = 0; j < NMAX; j += 4) {
                d0 = fmaf(ST[j], gs.a[p][j], d0);
                d1 = fmaf(ST[j + 1], gs.a[p][j + 1], d1);
                d2 = fmaf(ST[j + 2], gs.a[p][j + 2], d2);
                d3 = fmaf(ST[j + 3], gs.a[p][j + 3], d3);
            }
            dr = (d0 + d1) + (d2 + d3);
        }

        const float idi = __fdividef(1.f, di);
        float dw = 0.f, dk = 0.f, dv = 0.f, db = 0.f, dSb = 0.f;
#pragma unroll
        for (int j = 0; j < NMAX; ++j) {
            const float vv = vs.a[p][j], sa = ss.a[p][j];
            ST[j] = (ST[j] - ki * vv - bi * sa) * idi;
            DR[j] = fmaf(gi, rs.a[p][j], DR[j]);
            DT[j] = fmaf(ri, gs.a[p][j], DT[j]);
            dw = fmaf(DT[j], ST[j], dw);
            dk = fmaf(DT[j], vv, dk);
            db = fmaf(DT[j], sa, db);
            dv = fmaf(DR[j], ks.a[p][j], dv);
            dSb = fmaf(DR[j], bs.a[p][j], dSb);
        }
        dsb[i] = dSb;
        __syncthreads();
        if (t >= kAhead && live) {   // the rows of a later token into L1: the loads below then find them there
            const i64 o = base + (i64)(t - kAhead) * C;
            if (line_lead) {
                prefetch_l1(r_ + o); prefetch_l1(w_ + o); prefetch_l1(k_ + o); prefetch_l1(v_ + o);
                prefetch_l1(a_ + o); prefetch_l1(b_ + o); prefetch_l1(dy_ + o);
            }
            if (line_lead_sa) prefetch_l1(sa_ + o);
        }
        if (t > 0 && live) {   // the next token, requested here: the registers it takes are not live in the loop above
            const i64 o = base + (i64)(t - 1) * C;
            rn = to_f(r_[o]); wn = to_f(w_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]);
            an = to_f(a_[o]); bn = to_f(b_[o]); gn = to_f(dy_[o]); sn = sa_[o];
        }
        float da;
        {
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int j = 0; j < NMAX; j += 4) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float x = dsb[j + q];
                    if (q == 0) a0 = fmaf(ST[j + q], x, a0);
                    if (q == 1) a1 = fmaf(ST[j + q], x, a1);
                    if (q == 2) a2 = fmaf(ST[j + q], x, a2);
                    if (q == 3) a3 = fmaf(ST[j + q], x, a3);
                    DR[j + q] = fmaf(DR[j + q], ds.a[p][j + q], dSb * as.a[p][j + q]);
                    DT[j + q] = fmaf(DT[j + q], di, ai * x);
                }
            }
            da = (a0 + a1) + (a2 + a3);
        }
        if (live) {
            const i64 o = base + (i64)t * C;
            dr_[o] = from_f<E>(dr);
            dw_[o] = from_f<E>(kWScale * dw * di * sig * (1.f - sig));
            dk_[o] = from_f<E>(dk);
            dv_[o] = from_f<E>(dv);
            da_[o] = from_f<E>(da);
            db_[o] = from_f<E>(db);
        }
    }
    if (ds0_ != nullptr && live) {
#pragma unroll
        for (int j = 0; j < NMAX; ++j)
            if (j < N) ds0_[sbase + (i64)i * N + j] = DR[j];
    }
}

}  // namespace

int wkv7_generic_forward(int dtype, int B, int T, int H, int N, int chunk, const float* s0, const void* r,
                         const void* w, const void* k, const void* v, const void* a, const void* b, void* y,
                         float* sT, float* s, float* sa, cudaStream_t st) {
    dim3 grid(H, B);
#define RWKV_GO(E, NM)                                                                                           \
    wkv7_forward_kernel<E, NM><<<grid, NM, 0, st>>>(T, H, N, chunk, s0, (const E*)r, (const E*)w, (const E*)k,   \
                                                     (const E*)v, (const E*)a, (const E*)b, (E*)y, sT, s, sa)
    const int cap = head_capacity(N);
    if (dtype == RWKVB200_F32) {
        if (cap == 32) RWKV_GO(float, 32); else if (cap == 64) RWKV_GO(float, 64); else RWKV_GO(float, 128);
    } else {
        if (cap == 32) RWKV_GO(bf16, 32); else if (cap == 64) RWKV_GO(bf16, 64); else RWKV_GO(bf16, 128);
    }
#undef RWKV_GO
    return check_launch("wkv7_forward");
}

int wkv7_generic_backward(int dtype, int B, int T, int H, int N, int chunk, const void* r, const void* w,
                          const void* k, const void* v, const void* a, const void* b, const void* dy,
                          const float* dsT, const float* s, const float* sa, float* ds0, void* dr, void* dw, void* dk,
                          void* dv, void* da, void* db, cudaStream_t st) {
    dim3 grid(H, B);
#define RWKV_GO(E, NM)                                                                                            \
    wkv7_backward_kernel<E, NM><<<grid, NM, 0, st>>>(T, H, N, chunk, (const E*)r, (const E*)w, (const E*)k,       \
                                                      (const E*)v, (const E*)a, (const E*)b, (const E*)dy, dsT, s, \
                                                      sa, ds0, (E*)dr, (E*)dw, (E*)dk, (E*)dv, (E*)da, (E*)db)
    const int cap = head_capacity(N);
    if (dtype == RWKVB200_F32) {
        if (cap == 32) RWKV_GO(float, 32); else if (cap == 64) RWKV_GO(float, 64); else RWKV_GO(float, 128);
    } else {
        if (cap == 32) RWKV_GO(bf16, 32); else if (cap == 64) RWKV_GO(bf16, 64); else RWKV_GO(bf16, 128);
    }
#undef RWKV_GO
    return check_launch("wkv7_backward");
}

}  // namespace rwkvb200
