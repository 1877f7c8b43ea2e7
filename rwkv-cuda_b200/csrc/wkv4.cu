// RWKV-4 WKV, fp32, forward and backward.
//
// Operator (wkv/run.py:34-63 of the reference project), per batch b and channel c:
//   y_t = (sum_{s<t} e^{(t-1-s)w+k_s} v_s + e^{u+k_t} v_t) / (sum_{s<t} e^{(t-1-s)w+k_s} + e^{u+k_t})
// One thread owns one (b,c) recurrence; adjacent threads own adjacent channels so every
// global access of a warp is one coalesced 128-byte line.  Running sums are kept divided by
// e^{o} (o = running maximum exponent) so nothing overflows.  Of each pair exp(x-max),
// exp(y-max) one is exactly 1, so a step costs two exponentials, not four.
//
// The backward needs y_t and log(den_t) of every step again in its reverse sweep.  Instead of
// a per-thread local array (which limits T and spills to DRAM) the forward sweep parks them
// in the thread's own slots of the gk / gv output buffers, and the reverse sweep reads each
// slot back just before overwriting it with the real gradient.  No scratch, no limit on T.
//
// Compiled without fast-math: the fp32 tolerance of this operator (1e-5) needs accurate expf.
#include "common.cuh"

namespace rwkvb200 {

namespace {

constexpr float kNegInf = -1e38f;
constexpr int kBlk = 8;  // tokens fetched ahead per thread

struct Pair {
    float a, b, m;
};
// returns a = e^{x-m}, b = e^{y-m}, m = max(x,y) with one exponential
__device__ __forceinline__ Pair softpair(float x, float y) {
    float d = x - y;
    float e = expf(-fabsf(d));
    Pair r;
    r.a = d >= 0.f ? 1.f : e;
    r.b = d >= 0.f ? e : 1.f;
    r.m = fmaxf(x, y);
    return r;
}

__global__ void __launch_bounds__(128) wkv4_forward_kernel(int B, int T, int C, const float* __restrict__ w_,
                                                          const float* __restrict__ u_, const float* __restrict__ k_,
                                                          const float* __restrict__ v_, float* __restrict__ y_) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * C) return;
    const int b = idx / C, c = idx - b * C;
    const i64 off = (i64)b * T * C + c;
    const float u = u_[c], w = w_[c];
    const float* __restrict__ k = k_ + off;
    const float* __restrict__ v = v_ + off;
    float* __restrict__ y = y_ + off;

    float p = 0.f, q = 0.f, o = kNegInf;
    float kb[kBlk], vb[kBlk];
#pragma unroll
    for (int i = 0; i < kBlk; ++i) {
        kb[i] = i < T ? k[(i64)i * C] : 0.f;
        vb[i] = i < T ? v[(i64)i * C] : 0.f;
    }
    for (int t0 = 0; t0 < T; t0 += kBlk) {
        float kn[kBlk], vn[kBlk];
#pragma unroll
        for (int i = 0; i < kBlk; ++i) {  // next block's loads are in flight during this block's math
            const int t = t0 + kBlk + i;
            kn[i] = t < T ? k[(i64)t * C] : 0.f;
            vn[i] = t < T ? v[(i64)t * C] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < kBlk; ++i) {
            const int t = t0 + i;
            if (t < T) {
                const float kt = kb[i], vt = vb[i];
                Pair s = softpair(o, u + kt);
                y[(i64)t * C] = (s.a * p + s.b * vt) / (s.a * q + s.b);
                s = softpair(w + o, kt);
                p = s.a * p + s.b * vt;
                q = s.a * q + s.b;
                o = s.m;
            }
        }
#pragma unroll
        for (int i = 0; i < kBlk; ++i) {
            kb[i] = kn[i];
            vb[i] = vn[i];
        }
    }
}

__global__ void __launch_bounds__(128) wkv4_backward_kernel(int B, int T, int C, const float* __restrict__ w_,
                                                           const float* __restrict__ u_, const float* __restrict__ k_,
                                                           const float* __restrict__ v_, const float* __restrict__ gy_,
                                                           float* __restrict__ gw_, float* __restrict__ gu_,
                                                           float* gk_, float* gv_) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * C) return;
    const int b = idx / C, c = idx - b * C;
    const i64 off = (i64)b * T * C + c;
    const float u = u_[c], w = w_[c];
    const float* __restrict__ k = k_ + off;
    const float* __restrict__ v = v_ + off;
    const float* __restrict__ gy = gy_ + off;
    float* gk = gk_ + off;  // forward sweep parks y_t here
    float* gv = gv_ + off;  // forward sweep parks log(den_t) here

    // ---- forward sweep: y_t, log den_t, gw, gu -----------------------------------------
    float p = 0.f, q = 0.f, dp = 0.f, dq = 0.f, o = kNegInf;
    float gw = 0.f, gu = 0.f;
#pragma unroll 4
    for (int t = 0; t < T; ++t) {
        const float kt = k[(i64)t * C], vt = v[(i64)t * C], gyt = gy[(i64)t * C];
        Pair s = softpair(o, u + kt);
        const float den = s.a * q + s.b;
        const float iden = 1.f / den;
        const float yt = (s.a * p + s.b * vt) * iden;
        gk[(i64)t * C] = yt;
        gv[(i64)t * C] = s.m + logf(den);
        gw += gyt * (dp - dq * yt) * iden * s.a;
        gu += gyt * (vt - yt) * s.b * iden;
        s = softpair(w + o, kt);
        dp = s.a * (p + dp);
        dq = s.a * (q + dq);
        p = s.a * p + s.b * vt;
        q = s.a * q + s.b;
        o = s.m;
    }
    // the chain rule through w = -exp(time_decay) is applied here, as the reference does
    gw_[(i64)b * C + c] += gw * w;
    gu_[(i64)b * C + c] += gu;

    // ---- reverse sweep: gk, gv ----------------------------------------------------------
    float gp = 0.f, gq = 0.f;
    o = kNegInf;
#pragma unroll 4
    for (int t = T - 1; t >= 0; --t) {
        const float kt = k[(i64)t * C], vt = v[(i64)t * C], gyt = gy[(i64)t * C];
        const float yt = gk[(i64)t * C];
        const float lden = gv[(i64)t * C];
        const float A = gyt * expf(u + kt - lden);
        const float Bk = expf(kt + o);
        gk[(i64)t * C] = A * (vt - yt) + Bk * (gp * vt + gq);
        gv[(i64)t * C] = A + Bk * gp;
        Pair s = softpair(w + o, -lden);
        const float g = gyt * s.b;
        gp = s.a * gp + g;
        gq = s.a * gq - g * yt;
        o = s.m;
    }
}

int launch_shape(int B, int C, int* block) {
    const i64 n = (i64)B * C;
    // few recurrences: spread them one warp per CTA over as many SMs as possible
    *block = n <= 148 * 4 * 32 ? 32 : 128;
    return (int)((n + *block - 1) / *block);
}

}  // namespace

}  // namespace rwkvb200

using namespace rwkvb200;

extern "C" int rwkvb200_wkv4_forward(int B, int T, int C, const float* w, const float* u, const float* k,
                                     const float* v, float* y, void* stream) {
    RWKV_REQUIRE(B > 0 && T > 0 && C > 0, RWKVB200_EINVAL, "wkv4_forward: B=%d T=%d C=%d must be positive", B, T, C);
    RWKV_REQUIRE((i64)B * C < (1ll << 31), RWKVB200_EINVAL, "wkv4_forward: B*C too large");
    RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(y);
    int block;
    const int grid = launch_shape(B, C, &block);
    wkv4_forward_kernel<<<grid, block, 0, as_stream(stream)>>>(B, T, C, w, u, k, v, y);
    return check_launch("wkv4_forward");
}

extern "C" int rwkvb200_wkv4_backward(int B, int T, int C, const float* w, const float* u, const float* k,
                                      const float* v, const float* gy, float* gw, float* gu, float* gk,
                                      float* gv, void* stream) {
    RWKV_REQUIRE(B > 0 && T > 0 && C > 0, RWKVB200_EINVAL, "wkv4_backward: B=%d T=%d C=%d must be positive", B, T, C);
    RWKV_REQUIRE((i64)B * C < (1ll << 31), RWKVB200_EINVAL, "wkv4_backward: B*C too large");
    RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(gy);
    RWKV_NOTNULL(gw); RWKV_NOTNULL(gu); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv);
    int block;
    const int grid = launch_shape(B, C, &block);
    wkv4_backward_kernel<<<grid, block, 0, as_stream(stream)>>>(B, T, C, w, u, k, v, gy, gw, gu, gk, gv);
    return check_launch("wkv4_backward");
}
