// RWKV-5 and RWKV-5a WKV (static per-channel decay), fp32 or bf16 activations, fp32 state.
//
// Operator (wkv5/run.py:66-87 and wkv5a/run.py:260-289 of the reference project), per (b,h):
//   y_t[i] = sum_j r_t[j] ( U[j,i] k_t[j] v_t[i] + S[j,i] ),   S[j,i] <- W[j,i] S[j,i] + k_t[j] v_t[i]
//   RWKV-5 : W[j,i] = w[j],        U[j,i] = u[j]
//   RWKV-5a: W[j,i] = w1[j] w2[i], U[j,i] = u1[j] + u2[i]
// (j = key channel, i = value channel, S starts at zero.)
//
// One CTA per (batch, head); thread x owns one line of the N x N state in registers and the
// per-token vectors it has to see from its neighbours are exchanged through a double-buffered
// shared-memory stage (one barrier per token); the next token's elements are already in
// registers while the current one is being processed.
//
// Backward, three sweeps over time with at most two state lines per thread:
//   1. forward, thread = key i:   S[i,:], Z[i,:]  -> gr, gu(1), gw(1)
//        Z_t = sum_{s<t} (t-1-s) W^{t-1-s} k_s v_s^T obeys Z <- W (Z + S), and
//        dL/dlog w[i] = sum_t r_t[i] sum_j gy_t[j] Z_t[i,j]: no scratch, no second pass.
//   1b (RWKV-5a only). forward, thread = value i: S[:,i], Z[:,i] -> gu2, gw2
//   2. reverse, thread = key i and value i at once: D[i,:] -> gk,  D[:,i] -> gv
// gw is returned multiplied by ww = -exp(w_raw), gw/gu as per-batch partials (B,C), exactly
// what the reference kernels hand to their autograd wrappers.
#include "common.cuh"
#include "wkv6_chunked.cuh"
#include "wkv6_tsplit.cuh"
#include <initializer_list>
#include <type_traits>

namespace rwkvb200 {
namespace {

template <int NMAX>
struct __align__(16) Stage {
    float a[2][NMAX];
};

// ------------------------------------------------------------------------------------
template <typename E, int NMAX, bool DUAL>
__global__ void __launch_bounds__(NMAX) wkv5_forward_kernel(int T, int C, int H, int N, const E* __restrict__ r_,
                                                           const E* __restrict__ k_, const E* __restrict__ v_,
                                                           const float* __restrict__ w1_, const E* __restrict__ u1_,
                                                           const float* __restrict__ w2_, const E* __restrict__ u2_,
                                                           E* __restrict__ y_, const int* __restrict__ only_if_) {
    if (only_if_ != nullptr && only_if_[blockIdx.x & (kChunkedFlagUnits - 1)] == 0) return;   // fallback launch: the chunked kernel's result stands for this unit
    const int b = blockIdx.x / H, h = blockIdx.x - b * H, i = threadIdx.x;
    const bool live = i < N;
    __shared__ Stage<NMAX> rs, ks;
    __shared__ __align__(16) float ws[NMAX], us[NMAX];
    ws[i] = live ? w1_[h * N + i] : 0.f;
    us[i] = live ? to_f(u1_[h * N + i]) : 0.f;
    const float w2 = (DUAL && live) ? w2_[h * N + i] : 1.f;
    const float u2 = (DUAL && live) ? to_f(u2_[h * N + i]) : 0.f;

    float S[NMAX];
#pragma unroll
    for (int j = 0; j < NMAX; ++j) S[j] = 0.f;

    const i64 base = (i64)b * T * C + h * N + i;
    float rn = live ? to_f(r_[base]) : 0.f, kn = live ? to_f(k_[base]) : 0.f, vn = live ? to_f(v_[base]) : 0.f;
    for (int t = 0; t < T; ++t) {
        const int p = t & 1;
        rs.a[p][i] = rn;
        ks.a[p][i] = kn;
        const float v = vn;
        __syncthreads();
        if (t + 1 < T && live) {
            const i64 o = base + (i64)(t + 1) * C;
            rn = to_f(r_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]);
        }
        float y = 0.f;
#pragma unroll
        for (int j = 0; j < NMAX; j += 4) {
            const float4 r4 = *reinterpret_cast<const float4*>(&rs.a[p][j]);
            const float4 k4 = *reinterpret_cast<const float4*>(&ks.a[p][j]);
            const float4 w4 = *reinterpret_cast<const float4*>(&ws[j]);
            const float4 u4 = *reinterpret_cast<const float4*>(&us[j]);
            const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
            const float ww[4] = {w4.x, w4.y, w4.z, w4.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x = kk[e] * v;
                y = fmaf(rr[e], fmaf(DUAL ? uu[e] + u2 : uu[e], x, S[j + e]), y);
                S[j + e] = fmaf(S[j + e], DUAL ? ww[e] * w2 : ww[e], x);
            }
        }
        if (live) y_[base + (i64)t * C] = from_f<E>(y);
    }
}

// ------------------------------------------------------------------------------------
template <typename E, int NMAX, bool DUAL>
__global__ void __launch_bounds__(NMAX) wkv5_backward_kernel(
    int T, int C, int H, int N, const E* __restrict__ r_, const E* __restrict__ k_, const E* __restrict__ v_,
    const float* __restrict__ w1_, const float* __restrict__ ww1_, const E* __restrict__ u1_,
    const float* __restrict__ w2_, const float* __restrict__ ww2_, const E* __restrict__ u2_,
    const E* __restrict__ gy_, E* __restrict__ gr_, E* __restrict__ gk_, E* __restrict__ gv_, E* __restrict__ gw1_,
    E* __restrict__ gu1_, E* __restrict__ gw2_, E* __restrict__ gu2_, const int* __restrict__ only_if_) {
    if (only_if_ != nullptr && only_if_[blockIdx.x & (kChunkedFlagUnits - 1)] == 0) return;   // fallback launch: the chunked kernels' result stands for this unit
    const int b = blockIdx.x / H, h = blockIdx.x - b * H, i = threadIdx.x;
    const bool live = i < N;
    __shared__ Stage<NMAX> rs, ks, vs, gs;
    __shared__ __align__(16) float w1s[NMAX], u1s[NMAX], w2s[NMAX], u2s[NMAX];
    w1s[i] = live ? w1_[h * N + i] : 0.f;
    u1s[i] = live ? to_f(u1_[h * N + i]) : 0.f;
    w2s[i] = (DUAL && live) ? w2_[h * N + i] : (live ? 1.f : 0.f);
    u2s[i] = (DUAL && live) ? to_f(u2_[h * N + i]) : 0.f;
    __syncthreads();
    const float w1 = w1s[i], u1 = u1s[i], w2 = w2s[i], u2 = u2s[i];
    const i64 base = (i64)b * T * C + h * N + i;
    const i64 pbase = (i64)b * C + h * N + i;

    float S[NMAX], Z[NMAX];

    // ---- sweep 1: thread = key i, lines over value j -----------------------------------
    {
#pragma unroll
        for (int j = 0; j < NMAX; ++j) S[j] = Z[j] = 0.f;
        float gu = 0.f, gw = 0.f;
        float rn = live ? to_f(r_[base]) : 0.f, kn = live ? to_f(k_[base]) : 0.f;
        float vn = live ? to_f(v_[base]) : 0.f, gn = live ? to_f(gy_[base]) : 0.f;
        for (int t = 0; t < T; ++t) {
            const int p = t & 1;
            vs.a[p][i] = vn;
            gs.a[p][i] = gn;
            const float r = rn, k = kn;
            __syncthreads();
            if (t + 1 < T && live) {
                const i64 o = base + (i64)(t + 1) * C;
                rn = to_f(r_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]); gn = to_f(gy_[o]);
            }
            float gr = 0.f, xg = 0.f, zg = 0.f;
#pragma unroll
            for (int j = 0; j < NMAX; ++j) {
                const float x = k * vs.a[p][j], g = gs.a[p][j];
                const float w = DUAL ? w1 * w2s[j] : w1;
                gr = fmaf(fmaf(DUAL ? u1 + u2s[j] : u1, x, S[j]), g, gr);
                xg = fmaf(x, g, xg);
                zg = fmaf(Z[j], g, zg);
                Z[j] = w * (Z[j] + S[j]);
                S[j] = fmaf(S[j], w, x);
            }
            if (live) gr_[base + (i64)t * C] = from_f<E>(gr);
            gu = fmaf(r, xg, gu);
            gw = fmaf(r, zg, gw);
        }
        if (live) {
            gu1_[pbase] = from_f<E>(gu);
            gw1_[pbase] = from_f<E>(ww1_[h * N + i] * gw);
        }
    }

    // ---- sweep 1b (RWKV-5a): thread = value i, lines over key j ------------------------
    if (DUAL) {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < NMAX; ++j) S[j] = Z[j] = 0.f;
        float gu = 0.f, gw = 0.f;
        float rn = live ? to_f(r_[base]) : 0.f, kn = live ? to_f(k_[base]) : 0.f;
        float vn = live ? to_f(v_[base]) : 0.f, gn = live ? to_f(gy_[base]) : 0.f;
        for (int t = 0; t < T; ++t) {
            const int p = t & 1;
            rs.a[p][i] = rn;
            ks.a[p][i] = kn;
            const float v = vn, g = gn;
            __syncthreads();
            if (t + 1 < T && live) {
                const i64 o = base + (i64)(t + 1) * C;
                rn = to_f(r_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]); gn = to_f(gy_[o]);
            }
            float rk = 0.f, zr = 0.f;
#pragma unroll
            for (int j = 0; j < NMAX; ++j) {
                const float x = v * ks.a[p][j], r = rs.a[p][j];
                const float w = w1s[j] * w2;
                rk = fmaf(r, ks.a[p][j], rk);
                zr = fmaf(Z[j], r, zr);
                Z[j] = w * (Z[j] + S[j]);
                S[j] = fmaf(S[j], w, x);
            }
            gu = fmaf(g * v, rk, gu);
            gw = fmaf(g, zr, gw);
        }
        if (live) {
            gu2_[pbase] = from_f<E>(gu);
            gw2_[pbase] = from_f<E>(ww2_[h * N + i] * gw);
        }
    }

    // ---- sweep 2: reverse; S = D[key i, :], Z = D[:, value i] --------------------------
    {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < NMAX; ++j) S[j] = Z[j] = 0.f;
        const i64 last = base + (i64)(T - 1) * C;
        float rn = live ? to_f(r_[last]) : 0.f, kn = live ? to_f(k_[last]) : 0.f;
        float vn = live ? to_f(v_[last]) : 0.f, gn = live ? to_f(gy_[last]) : 0.f;
        for (int t = T - 1; t >= 0; --t) {
            const int p = t & 1;
            rs.a[p][i] = rn; ks.a[p][i] = kn; vs.a[p][i] = vn; gs.a[p][i] = gn;
            const float r = rn, g = gn;
            __syncthreads();
            if (t > 0 && live) {
                const i64 o = base + (i64)(t - 1) * C;
                rn = to_f(r_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]); gn = to_f(gy_[o]);
            }
            float gk = 0.f, gv = 0.f;
#pragma unroll
            for (int j = 0; j < NMAX; ++j) {
                const float x = r * gs.a[p][j];    // key i, value j
                const float x2 = g * rs.a[p][j];   // key j, value i
                const float wa = DUAL ? w1 * w2s[j] : w1;
                const float wb = DUAL ? w1s[j] * w2 : w1s[j];
                gk = fmaf(fmaf(DUAL ? u1 + u2s[j] : u1, x, S[j]), vs.a[p][j], gk);
                gv = fmaf(fmaf(DUAL ? u1s[j] + u2 : u1s[j], x2, Z[j]), ks.a[p][j], gv);
                S[j] = fmaf(S[j], wa, x);
                Z[j] = fmaf(Z[j], wb, x2);
            }
            if (live) {
                gk_[base + (i64)t * C] = from_f<E>(gk);
                gv_[base + (i64)t * C] = from_f<E>(gv);
            }
        }
    }
}

template <typename E>
bool chunked_ok(int T, int N, std::initializer_list<const void*> ps) {
    if (!std::is_same<E, bf16>::value || N != 64 || T % 16 != 0) return false;
    for (const void* p : ps)
        if (p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) != 0) return false;
    return true;
}

template <typename E, bool DUAL>
int launch_fwd(int B, int T, int C, int H, const void* r, const void* k, const void* v, const float* w1,
               const void* u1, const float* w2, const void* u2, void* y, cudaStream_t st) {
    const int N = C / H;
    const int* only_if = nullptr;
    if (!DUAL && chunked_ok<E>(T, N, {r, k, v, u1, y})) {
        // RWKV-5 is RWKV-6 with a decay that does not change over time: the chunked tensor-core kernel
        // runs first, the general-shape kernel below only if the decay is too strong for the chunked form
        int* flag = wkv6_chunked_flag(st);   // NULL: every slot is taken, the general-shape kernel runs alone
        if (flag != nullptr) {
            RWKV_REQUIRE(cudaMemsetAsync(flag, 0, sizeof(int) * kChunkedFlagUnits, st) == cudaSuccess, RWKVB200_ECUDA, "wkv5_forward: clearing the device flag failed");
            if (int e = wkv6_chunked_forward(B, T, H, r, k, v, w1, 2, u1, nullptr, 0, y, nullptr, nullptr, flag, st)) return e;
            only_if = flag;
        }
    }
#define RWKV_GO(NM)                                                                                           \
    wkv5_forward_kernel<E, NM, DUAL><<<B * H, NM, 0, st>>>(T, C, H, N, (const E*)r, (const E*)k, (const E*)v, \
                                                            w1, (const E*)u1, w2, (const E*)u2, (E*)y, only_if)
    switch (head_capacity(N)) {
        case 32: RWKV_GO(32); break;
        case 64: RWKV_GO(64); break;
        default: RWKV_GO(128); break;
    }
#undef RWKV_GO
    return check_launch(DUAL ? "wkv5a_forward" : "wkv5_forward");
}

// fp32 copies of the (B,C) partials; only_if: run only when that device flag is set (NULL: always)
template <typename E>
__global__ void widen_partials_kernel(int n, int C, int N, const E* __restrict__ gw, const E* __restrict__ gu,
                                      float* __restrict__ gw32, float* __restrict__ gu32, const int* __restrict__ only_if) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int unit = (i / C) * (C / N) + (i % C) / N;   // (batch, head) of this element
    if (only_if != nullptr && only_if[unit & (kChunkedFlagUnits - 1)] == 0) return;
    gw32[i] = to_f(gw[i]); gu32[i] = to_f(gu[i]);
}

template <typename E, bool DUAL>
int launch_bwd(int B, int T, int C, int H, const void* r, const void* k, const void* v, const float* w1,
               const float* ww1, const void* u1, const float* w2, const float* ww2, const void* u2, const void* gy,
               void* gr, void* gk, void* gv, void* gw1, void* gu1, void* gw2, void* gu2, cudaStream_t st,
               void* scratch = nullptr, float* gw32 = nullptr, float* gu32 = nullptr) {
    const int N = C / H;
    const int* only_if = nullptr;
    if (!DUAL && scratch != nullptr && chunked_ok<E>(T, N, {r, k, v, u1, gy, gr, gk, gv, gw1, gu1, scratch})) {
        // chunked forward into the scratch buffer (chunk-start states), chunked reverse pass, then the
        // general-shape kernel only if the decay is too strong for the chunked form
        int* flag = wkv6_chunked_flag(st);   // NULL: every slot is taken, the general-shape kernel runs alone
        if (flag != nullptr) {
            RWKV_REQUIRE(cudaMemsetAsync(flag, 0, sizeof(int) * kChunkedFlagUnits, st) == cudaSuccess, RWKVB200_ECUDA, "wkv5_backward: clearing the device flag failed");
            float* ck = static_cast<float*>(scratch);
            if (int e = wkv6_backward_with_states(B, T, H, r, k, v, ww1, 3, u1, nullptr, 0, gy, nullptr, ck, gr, gk, gv, gw1, gu1,
                                                  nullptr, 0, flag, st, gw32, gu32))
                return e;
            only_if = flag;
        }
    }
#define RWKV_GO(NM)                                                                                              \
    wkv5_backward_kernel<E, NM, DUAL><<<B * H, NM, 0, st>>>(                                                     \
        T, C, H, N, (const E*)r, (const E*)k, (const E*)v, w1, ww1, (const E*)u1, w2, ww2, (const E*)u2,         \
        (const E*)gy, (E*)gr, (E*)gk, (E*)gv, (E*)gw1, (E*)gu1, (E*)gw2, (E*)gu2, only_if)
    switch (head_capacity(N)) {
        case 32: RWKV_GO(32); break;
        case 64: RWKV_GO(64); break;
        default: RWKV_GO(128); break;
    }
#undef RWKV_GO
    if (gw32 != nullptr && gu32 != nullptr) {
        // the general-shape kernel has the (B,C) partials in the activation type only: where it ran (it was the
        // only kernel, or the chunked one raised its flag) the fp32 copies are made from those
        widen_partials_kernel<E><<<(B * C + 255) / 256, 256, 0, st>>>(B * C, C, N, (const E*)gw1, (const E*)gu1, gw32, gu32, only_if);
    }
    return check_launch(DUAL ? "wkv5a_backward" : "wkv5_backward");
}

int check_dims(const char* what, int dtype, int B, int T, int C, int H) {
    RWKV_REQUIRE(dtype == RWKVB200_F32 || dtype == RWKVB200_BF16, RWKVB200_EINVAL, "%s: unknown dtype %d", what, dtype);
    RWKV_REQUIRE(B > 0 && T > 0 && C > 0 && H > 0, RWKVB200_EINVAL, "%s: B=%d T=%d C=%d H=%d must be positive", what, B, T, C, H);
    RWKV_REQUIRE(C % H == 0, RWKVB200_EINVAL, "%s: C=%d is not a multiple of H=%d", what, C, H);
    RWKV_REQUIRE(C / H <= RWKVB200_MAX_HEAD_SIZE, RWKVB200_EUNSUPPORTED, "%s: head size %d > %d", what, C / H,
                 RWKVB200_MAX_HEAD_SIZE);
    return RWKVB200_OK;
}

}  // namespace
}  // namespace rwkvb200

using namespace rwkvb200;

extern "C" int rwkvb200_wkv5_forward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                     const void* v, const float* w, const void* u, void* y, void* stream) {
    if (int e = check_dims("wkv5_forward", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(y);
    return dtype == RWKVB200_F32
               ? launch_fwd<float, false>(B, T, C, H, r, k, v, w, u, nullptr, nullptr, y, as_stream(stream))
               : launch_fwd<bf16, false>(B, T, C, H, r, k, v, w, u, nullptr, nullptr, y, as_stream(stream));
}

// The forward split over time (wkv6_tsplit.cu; the reference's wkv5_bf16/cuda/wkv5_cuda_v3.cu is the same idea):
// `segments` pieces of T/segments tokens run at the same time.  Tensor-core shapes only (bf16, head size 64,
// T/segments a multiple of 16, 16-byte aligned tensors).  work: rwkvb200_wkv6_tsplit_bytes(B,T,C,H,segments) bytes.
extern "C" int rwkvb200_wkv5_forward_tsplit(int dtype, int B, int T, int C, int H, int segments, const void* r,
                                            const void* k, const void* v, const float* w, const void* u, void* y,
                                            void* work, void* stream) {
    if (int e = check_dims("wkv5_forward_tsplit", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(y); RWKV_NOTNULL(work);
    const int K = segments, N = C / H;
    RWKV_REQUIRE(K >= 1 && T % K == 0 && (T / K) % 16 == 0, RWKVB200_EINVAL,
                 "wkv5_forward_tsplit: T = %d is not %d segments of a multiple of 16 tokens", T, K);
    RWKV_REQUIRE(dtype == RWKVB200_BF16 && chunked_ok<bf16>(T / K, N, {r, k, v, u, y, work}), RWKVB200_EINVAL,
                 "wkv5_forward_tsplit: needs bf16 tensors, head size 64, 16-byte alignment");
    cudaStream_t st = as_stream(stream);
    int* flag = wkv6_chunked_flag(st);
    if (flag == nullptr || K == 1)   // no flag word left for this stream, or nothing to split: the plain forward
        return launch_fwd<bf16, false>(B, T, C, H, r, k, v, w, u, nullptr, nullptr, y, st);
    RWKV_REQUIRE(cudaMemsetAsync(flag, 0, sizeof(int) * kChunkedFlagUnits, st) == cudaSuccess, RWKVB200_ECUDA,
                 "wkv5_forward_tsplit: clearing the device flag failed");
    float* wk = static_cast<float*>(work);
    float* start = wk + (size_t)B * K * H * N * N;
    // 1. every segment from a zero state, states only  2. segment start states  3. every segment with its start state
    if (int e = wkv6_chunked_forward(B * K, T / K, H, r, k, v, w, 2, u, nullptr, 0, nullptr, wk, nullptr, flag, st, K)) return e;
    if (int e = wkv6_tsplit_states(B, T, C, H, K, w, 2, nullptr, wk, nullptr, st)) return e;
    if (int e = wkv6_chunked_forward(B * K, T / K, H, r, k, v, w, 2, u, start, 2, y, nullptr, nullptr, flag, st, K)) return e;
    // a decay too strong for the chunked form: the general-shape kernel redoes the call
    wkv5_forward_kernel<bf16, 64, false><<<B * H, 64, 0, st>>>(T, C, H, N, (const bf16*)r, (const bf16*)k, (const bf16*)v, w,
                                                              (const bf16*)u, nullptr, nullptr, (bf16*)y, flag);
    return check_launch("wkv5_forward_tsplit");
}

extern "C" int rwkvb200_wkv5_backward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                      const void* v, const float* w, const float* ww, const void* u, const void* gy,
                                      void* gr, void* gk, void* gv, void* gw, void* gu, void* stream) {
    if (int e = check_dims("wkv5_backward", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(ww); RWKV_NOTNULL(u);
    RWKV_NOTNULL(gy); RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu);
    return dtype == RWKVB200_F32
               ? launch_bwd<float, false>(B, T, C, H, r, k, v, w, ww, u, nullptr, nullptr, nullptr, gy, gr, gk, gv,
                                          gw, gu, nullptr, nullptr, as_stream(stream))
               : launch_bwd<bf16, false>(B, T, C, H, r, k, v, w, ww, u, nullptr, nullptr, nullptr, gy, gr, gk, gv,
                                         gw, gu, nullptr, nullptr, as_stream(stream));
}

extern "C" size_t rwkvb200_wkv5_scratch_bytes(int B, int T, int C) {
    if (B <= 0 || T <= 0 || C <= 0) return 0;
    return (size_t)B * T * C * sizeof(float) * 4;   // one fp32 64x64 state per 16 tokens and head
}

extern "C" int rwkvb200_wkv5_backward_ws(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                         const void* v, const float* w, const float* ww, const void* u,
                                         const void* gy, void* gr, void* gk, void* gv, void* gw, void* gu,
                                         void* scratch, void* stream) {
    if (int e = check_dims("wkv5_backward_ws", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(ww); RWKV_NOTNULL(u);
    RWKV_NOTNULL(gy); RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu);
    RWKV_NOTNULL(scratch);
    return dtype == RWKVB200_F32
               ? launch_bwd<float, false>(B, T, C, H, r, k, v, w, ww, u, nullptr, nullptr, nullptr, gy, gr, gk, gv,
                                          gw, gu, nullptr, nullptr, as_stream(stream), scratch)
               : launch_bwd<bf16, false>(B, T, C, H, r, k, v, w, ww, u, nullptr, nullptr, nullptr, gy, gr, gk, gv,
                                         gw, gu, nullptr, nullptr, as_stream(stream), scratch);
}

// As rwkvb200_wkv5_backward_ws, and in addition the (B,C) partials of gw and gu unrounded in fp32 (gw32, gu32):
// summed over the batch with rwkvb200_reduce_batch_partials they give the parameter gradients without the
// bf16 round trip of the reference harness (wkv5_bf16/run.py:83-87).
extern "C" int rwkvb200_wkv5_backward_ws32(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                           const void* v, const float* w, const float* ww, const void* u,
                                           const void* gy, void* gr, void* gk, void* gv, void* gw, void* gu,
                                           float* gw32, float* gu32, void* scratch, void* stream) {
    if (int e = check_dims("wkv5_backward_ws32", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(ww); RWKV_NOTNULL(u);
    RWKV_NOTNULL(gy); RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu);
    RWKV_NOTNULL(gw32); RWKV_NOTNULL(gu32); RWKV_NOTNULL(scratch);
    return dtype == RWKVB200_F32
               ? launch_bwd<float, false>(B, T, C, H, r, k, v, w, ww, u, nullptr, nullptr, nullptr, gy, gr, gk, gv,
                                          gw, gu, nullptr, nullptr, as_stream(stream), scratch, gw32, gu32)
               : launch_bwd<bf16, false>(B, T, C, H, r, k, v, w, ww, u, nullptr, nullptr, nullptr, gy, gr, gk, gv,
                                         gw, gu, nullptr, nullptr, as_stream(stream), scratch, gw32, gu32);
}

// Training flow with saved states (see rwkvb200_wkv6state_forward_saved): the forward leaves the states at the start
// of every 32-token chunk and the flags of its units in `saved` (rwkvb200_wkv5_scratch_bytes(B,T,C) bytes), the
// backward uses them.  The forward returns RWKVB200_OK when it saved them, 1 when not (pass saved_valid = 0).
// The backward also returns the unrounded fp32 (B,C) partials of gw and gu when gw32 / gu32 are given (both or none).
extern "C" int rwkvb200_wkv5_forward_saved(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                           const void* v, const float* w, const void* u, void* y, void* saved, void* stream) {
    if (int e = check_dims("wkv5_forward_saved", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(y); RWKV_NOTNULL(saved);
    const int N = C / H;
    cudaStream_t st = as_stream(stream);
    int* flag = nullptr;
    if (dtype == RWKVB200_BF16 && wkv6_forward_choice() && chunked_ok<bf16>(T, N, {r, k, v, u, y, saved})) flag = wkv6_chunked_flag(st);
    if (flag != nullptr) {
        RWKV_REQUIRE(cudaMemsetAsync(flag, 0, sizeof(int) * kChunkedFlagUnits, st) == cudaSuccess, RWKVB200_ECUDA,
                     "wkv5_forward_saved: clearing the device flags failed");
        const int rc = wkv6_l32_forward(B, T, H, r, k, v, w, 2, u, nullptr, 0, y, nullptr, static_cast<float*>(saved), flag, st, 1);
        if (rc < 0) return rc;
        if (rc == 0) {
            wkv5_forward_kernel<bf16, 64, false><<<B * H, 64, 0, st>>>(T, C, H, N, (const bf16*)r, (const bf16*)k, (const bf16*)v, w,
                                                                      (const bf16*)u, nullptr, nullptr, (bf16*)y, flag);
            if (int e = check_launch("wkv5_forward_saved")) return e;
            char* tail = static_cast<char*>(saved) + rwkvb200_wkv5_scratch_bytes(B, T, C) - sizeof(int) * kChunkedFlagUnits;
            RWKV_REQUIRE(cudaMemcpyAsync(tail, flag, sizeof(int) * kChunkedFlagUnits, cudaMemcpyDeviceToDevice, st) == cudaSuccess,
                         RWKVB200_ECUDA, "wkv5_forward_saved: saving the device flags failed");
            return RWKVB200_OK;
        }
    }
    const int e = dtype == RWKVB200_F32 ? launch_fwd<float, false>(B, T, C, H, r, k, v, w, u, nullptr, nullptr, y, st)
                                        : launch_fwd<bf16, false>(B, T, C, H, r, k, v, w, u, nullptr, nullptr, y, st);
    return e ? e : 1;
}

extern "C" int rwkvb200_wkv5_backward_saved(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                            const void* v, const float* w, const float* ww, const void* u, const void* gy,
                                            void* gr, void* gk, void* gv, void* gw, void* gu, float* gw32, float* gu32,
                                            void* saved, int saved_valid, void* stream) {
    if (int e = check_dims("wkv5_backward_saved", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(ww); RWKV_NOTNULL(u);
    RWKV_NOTNULL(gy); RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu); RWKV_NOTNULL(saved);
    RWKV_REQUIRE((gw32 == nullptr) == (gu32 == nullptr), RWKVB200_EINVAL, "wkv5_backward_saved: gw32 and gu32 go together");
    const int N = C / H;
    cudaStream_t st = as_stream(stream);
    int* flag = nullptr;
    if (saved_valid && dtype == RWKVB200_BF16 && chunked_ok<bf16>(T, N, {r, k, v, u, gy, gr, gk, gv, gw, gu, saved})) flag = wkv6_chunked_flag(st);
    if (flag != nullptr) {
        const char* tail = static_cast<const char*>(saved) + rwkvb200_wkv5_scratch_bytes(B, T, C) - sizeof(int) * kChunkedFlagUnits;
        RWKV_REQUIRE(cudaMemcpyAsync(flag, tail, sizeof(int) * kChunkedFlagUnits, cudaMemcpyDeviceToDevice, st) == cudaSuccess,
                     RWKVB200_ECUDA, "wkv5_backward_saved: restoring the device flags failed");
        if (int e = wkv6_l32_backward(B, T, H, r, k, v, ww, 3, u, gy, nullptr, static_cast<const float*>(saved), gr, gk, gv, gw, gu,
                                      nullptr, 0, st, gw32, gu32))
            return e;
        wkv5_backward_kernel<bf16, 64, false><<<B * H, 64, 0, st>>>(T, C, H, N, (const bf16*)r, (const bf16*)k, (const bf16*)v, w, ww,
                                                                   (const bf16*)u, nullptr, nullptr, nullptr, (const bf16*)gy,
                                                                   (bf16*)gr, (bf16*)gk, (bf16*)gv, (bf16*)gw, (bf16*)gu, nullptr,
                                                                   nullptr, flag);
        if (gw32 != nullptr)
            widen_partials_kernel<bf16><<<(B * C + 255) / 256, 256, 0, st>>>(B * C, C, N, (const bf16*)gw, (const bf16*)gu, gw32, gu32, flag);
        return check_launch("wkv5_backward_saved");
    }
    return dtype == RWKVB200_F32
               ? launch_bwd<float, false>(B, T, C, H, r, k, v, w, ww, u, nullptr, nullptr, nullptr, gy, gr, gk, gv, gw, gu, nullptr,
                                          nullptr, st, saved, gw32, gu32)
               : launch_bwd<bf16, false>(B, T, C, H, r, k, v, w, ww, u, nullptr, nullptr, nullptr, gy, gr, gk, gv, gw, gu, nullptr,
                                         nullptr, st, saved, gw32, gu32);
}

extern "C" int rwkvb200_wkv5a_forward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                      const void* v, const float* w1, const void* u1, const float* w2,
                                      const void* u2, void* y, void* stream) {
    if (int e = check_dims("wkv5a_forward", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w1); RWKV_NOTNULL(u1); RWKV_NOTNULL(w2);
    RWKV_NOTNULL(u2); RWKV_NOTNULL(y);
    return dtype == RWKVB200_F32 ? launch_fwd<float, true>(B, T, C, H, r, k, v, w1, u1, w2, u2, y, as_stream(stream))
                                 : launch_fwd<bf16, true>(B, T, C, H, r, k, v, w1, u1, w2, u2, y, as_stream(stream));
}

extern "C" int rwkvb200_wkv5a_backward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                       const void* v, const float* w1, const float* ww1, const void* u1,
                                       const float* w2, const float* ww2, const void* u2, const void* gy, void* gr,
                                       void* gk, void* gv, void* gw1, void* gu1, void* gw2, void* gu2, void* stream) {
    if (int e = check_dims("wkv5a_backward", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w1); RWKV_NOTNULL(ww1); RWKV_NOTNULL(u1);
    RWKV_NOTNULL(w2); RWKV_NOTNULL(ww2); RWKV_NOTNULL(u2); RWKV_NOTNULL(gy); RWKV_NOTNULL(gr); RWKV_NOTNULL(gk);
    RWKV_NOTNULL(gv); RWKV_NOTNULL(gw1); RWKV_NOTNULL(gu1); RWKV_NOTNULL(gw2); RWKV_NOTNULL(gu2);
    return dtype == RWKVB200_F32
               ? launch_bwd<float, true>(B, T, C, H, r, k, v, w1, ww1, u1, w2, ww2, u2, gy, gr, gk, gv, gw1, gu1,
                                         gw2, gu2, as_stream(stream))
               : launch_bwd<bf16, true>(B, T, C, H, r, k, v, w1, ww1, u1, w2, ww2, u2, gy, gr, gk, gv, gw1, gu1,
                                        gw2, gu2, as_stream(stream));
}

// ---- parameter gradients: per-batch partials -> one fp32 vector ------------------------------------------
namespace rwkvb200 {
namespace {
// out[off + j] = sum_b partial[b][j], fp32 accumulation in batch order (deterministic); one thread per column
template <typename E>
__global__ void reduce_batch_partials_kernel(int B, int n, const E* __restrict__ partial, float* __restrict__ out) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    float acc = 0.f;
    for (int b = 0; b < B; ++b) acc += to_f(partial[(i64)b * n + j]);
    out[j] = acc;
}
}  // namespace
}  // namespace rwkvb200

extern "C" int rwkvb200_reduce_batch_partials(int dtype, int B, int n, const void* partial, float* out, void* stream) {
    RWKV_REQUIRE(dtype == RWKVB200_F32 || dtype == RWKVB200_BF16, RWKVB200_EINVAL, "reduce_batch_partials: unknown dtype %d", dtype);
    RWKV_REQUIRE(B > 0 && n > 0, RWKVB200_EINVAL, "reduce_batch_partials: B=%d n=%d must be positive", B, n);
    RWKV_NOTNULL(partial); RWKV_NOTNULL(out);
    const int threads = 128, blocks = (n + threads - 1) / threads;
    if (dtype == RWKVB200_F32)
        reduce_batch_partials_kernel<float><<<blocks, threads, 0, as_stream(stream)>>>(B, n, (const float*)partial, out);
    else
        reduce_batch_partials_kernel<bf16><<<blocks, threads, 0, as_stream(stream)>>>(B, n, (const bf16*)partial, out);
    return check_launch("reduce_batch_partials");
}
