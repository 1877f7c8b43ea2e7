// depthwise_conv1d ("TimeX"): causal depthwise convolution with a full-length per-channel
// filter, fp32, forward and backward.
//
// Operator (depthwise_conv1d/run.py:41-55 of the reference project):
//   x[b,c,t]  = eps + sum_{u<=t} w[c,(T-1)-(t-u)] k[b,c,u]
//   gw[b,c,t] =       sum_{u<=t} g[b,c,(T-1)-(t-u)] k[b,c,u]           (then summed over b)
//   gk[b,c,u] =       sum_{t>=u} g[b,c,t] w[c,(T-1)-(t-u)]
// All three are the same causal correlation  out[t] = sum_{u<=t} F[(T-1)-t+u] G[u]:
//   forward: F = w[c] (shared by the batch), G = k[b,c]
//   gw     : F = g[b,c] (one per batch),     G = k[b,c]
//   gk     : F = w[c], G = g[b,c] read back to front, and the output written back to front.
// so one kernel template serves them.
//
// Mapping: one CTA per (channel, group of BG batch rows).  The filter row(s) and the BG
// signal rows are staged once in shared memory (zero padded to a multiple of 4 plus a 4-float
// zero tail so the triangular edge needs no special case).  A thread owns tiles of 4
// consecutive outputs x BG batch rows in registers and walks u in steps of 4 with 128-bit
// shared-memory reads: 2 reads of the filter window (conflict free: neighbouring threads read
// neighbouring float4s) and BG broadcast reads of the signals feed 16*BG FMAs.  The work of a
// tile grows linearly with t, so every thread takes tile p and its mirror image P-1-p: all
// threads do the same amount of work.  The binding roof of this operator is the FP32 pipe
// (T/2 FMAs per loaded element), not HBM.
#include "common.cuh"

namespace rwkvb200 {
namespace {

enum { kFwd = 0, kGk = 1, kGw = 2 };

template <int MODE, int BG>
__global__ void __launch_bounds__(1024) timex_kernel(const float* __restrict__ F_, const float* __restrict__ G_,
                                                    float* __restrict__ out, float eps, int B, int C, int T,
                                                    int Tp, int vec_ok) {
    extern __shared__ float4 smem4[];
    float* smem = reinterpret_cast<float*>(smem4);
    constexpr bool kFilterPerBatch = MODE >= kGw;
    constexpr int NF = kFilterPerBatch ? BG : 1;
    const int FS = Tp + 4;  // filter row stride, floats
    float* Fs = smem;
    float* Gs = smem + NF * FS;
    const int c = blockIdx.x, b0 = blockIdx.y * BG;
    const int pad = Tp - T;
    const int tid = threadIdx.x, nth = blockDim.x;

    for (int x = tid; x < FS; x += nth) {
        const bool in = x >= pad && x < Tp;
        if (!kFilterPerBatch) {
            Fs[x] = in ? F_[(i64)c * T + (x - pad)] : 0.f;
        } else {
#pragma unroll
            for (int j = 0; j < BG; ++j) {
                const int b = b0 + j;
                Fs[j * FS + x] = (in && b < B) ? F_[((i64)b * C + c) * T + (x - pad)] : 0.f;
            }
        }
    }
    for (int x = tid; x < Tp; x += nth) {
        const int src = MODE == kGk ? T - 1 - x : x;
#pragma unroll
        for (int j = 0; j < BG; ++j) {
            const int b = b0 + j;
            Gs[j * Tp + x] = (x < T && b < B) ? G_[((i64)b * C + c) * T + src] : 0.f;
        }
    }
    __syncthreads();

    const int P = Tp >> 2;
    const float init = MODE == kFwd ? eps : 0.f;
    for (int pp = tid; pp < (P + 1) / 2; pp += nth) {
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
            const int p = half == 0 ? pp : P - 1 - pp;
            if (half == 1 && p == pp) break;
            const int t0 = p << 2;
            float acc[BG][4];
#pragma unroll
            for (int j = 0; j < BG; ++j)
#pragma unroll
                for (int d = 0; d < 4; ++d) acc[j][d] = init;

            const float4* G4 = reinterpret_cast<const float4*>(Gs);
            const int fbase4 = (Tp - 4 - t0) >> 2;
            for (int q = 0; q <= p; ++q) {
                float f[8];
                if (!kFilterPerBatch) {
                    const float4* F4 = reinterpret_cast<const float4*>(Fs) + fbase4 + q;
                    const float4 f0 = F4[0], f1 = F4[1];
                    f[0] = f0.x; f[1] = f0.y; f[2] = f0.z; f[3] = f0.w;
                    f[4] = f1.x; f[5] = f1.y; f[6] = f1.z; f[7] = f1.w;
                }
#pragma unroll
                for (int j = 0; j < BG; ++j) {
                    if (kFilterPerBatch) {
                        const float4* F4 = reinterpret_cast<const float4*>(Fs + j * FS) + fbase4 + q;
                        const float4 f0 = F4[0], f1 = F4[1];
                        f[0] = f0.x; f[1] = f0.y; f[2] = f0.z; f[3] = f0.w;
                        f[4] = f1.x; f[5] = f1.y; f[6] = f1.z; f[7] = f1.w;
                    }
                    const float4 g4 = G4[j * (Tp >> 2) + q];
                    const float g[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
                    for (int uu = 0; uu < 4; ++uu)
#pragma unroll
                        for (int d = 0; d < 4; ++d) acc[j][d] = fmaf(f[3 - d + uu], g[uu], acc[j][d]);
                }
            }

            {
#pragma unroll
                for (int j = 0; j < BG; ++j) {
                    const int b = b0 + j;
                    if (b >= B) continue;
                    float* row = out + ((i64)b * C + c) * T;
                    if (vec_ok && t0 + 3 < T) {
                        if (MODE == kGk)
                            *reinterpret_cast<float4*>(row + (T - 4 - t0)) =
                                make_float4(acc[j][3], acc[j][2], acc[j][1], acc[j][0]);
                        else
                            *reinterpret_cast<float4*>(row + t0) =
                                make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
                    } else {
#pragma unroll
                        for (int d = 0; d < 4; ++d)
                            if (t0 + d < T) row[MODE == kGk ? T - 1 - (t0 + d) : t0 + d] = acc[j][d];
                    }
                }
            }
        }
    }
}

template <int MODE, int BG>
int launch(const float* F, const float* G, float* out, float eps, int B, int C, int T, cudaStream_t st,
           const char* what) {
    const int Tp = (T + 3) & ~3;
    constexpr int NF = MODE >= kGw ? BG : 1;
    const size_t smem = ((size_t)NF * (Tp + 4) + (size_t)BG * Tp) * sizeof(float);
    RWKV_REQUIRE(smem <= 227 * 1024, RWKVB200_EUNSUPPORTED, "%s: T=%d needs %zu bytes of shared memory (max 232448)",
                 what, T, smem);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(timex_kernel<MODE, BG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        RWKV_REQUIRE(e == cudaSuccess, RWKVB200_ECUDA, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(e));
    }
    const int P = Tp >> 2;
    int threads = ((P + 1) / 2 + 31) & ~31;
    if (threads > 1024) threads = 1024;
    const int vec_ok = (T % 4 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    dim3 grid(C, (B + BG - 1) / BG);
    timex_kernel<MODE, BG><<<grid, threads, smem, st>>>(F, G, out, eps, B, C, T, Tp, vec_ok);
    return check_launch(what);
}

// picks the widest batch group whose rows fit in shared memory
template <int MODE>
int launch_any(const float* F, const float* G, float* out, float eps, int B, int C, int T, cudaStream_t st,
               const char* what) {
    const int Tp = (T + 3) & ~3;
    auto fits = [&](int bg) {
        const int nf = MODE >= kGw ? bg : 1;
        return ((size_t)nf * (Tp + 4) + (size_t)bg * Tp) * sizeof(float) <= 100 * 1024;
    };
    if (MODE < kGw && B >= 8 && fits(8)) return launch<MODE, 8>(F, G, out, eps, B, C, T, st, what);
    if (B >= 4 && fits(4)) return launch<MODE, 4>(F, G, out, eps, B, C, T, st, what);
    if (B >= 2 && fits(2)) return launch<MODE, 2>(F, G, out, eps, B, C, T, st, what);
    return launch<MODE, 1>(F, G, out, eps, B, C, T, st, what);
}

int check_dims(int B, int C, int T, const char* what) {
    RWKV_REQUIRE(B > 0 && C > 0 && T > 0, RWKVB200_EINVAL, "%s: B=%d C=%d T=%d must be positive", what, B, C, T);
    RWKV_REQUIRE(B <= 65535 * 1, RWKVB200_EINVAL, "%s: B=%d too large", what, B);
    return RWKVB200_OK;
}

}  // namespace
}  // namespace rwkvb200

using namespace rwkvb200;

extern "C" int rwkvb200_timex_forward(const float* w, const float* k, float* x, float eps, int B, int C, int T,
                                      void* stream) {
    if (int e = check_dims(B, C, T, "timex_forward")) return e;
    RWKV_NOTNULL(w); RWKV_NOTNULL(k); RWKV_NOTNULL(x);
    return launch_any<kFwd>(w, k, x, eps, B, C, T, as_stream(stream), "timex_forward");
}

extern "C" int rwkvb200_timex_backward(const float* w, const float* k, const float* gwk, float* gw, float* gk,
                                       int B, int C, int T, void* stream) {
    if (int e = check_dims(B, C, T, "timex_backward")) return e;
    RWKV_NOTNULL(w); RWKV_NOTNULL(k); RWKV_NOTNULL(gwk); RWKV_NOTNULL(gw); RWKV_NOTNULL(gk);
    if (int e = launch_any<kGw>(gwk, k, gw, 0.f, B, C, T, as_stream(stream), "timex_backward(gw)")) return e;
    return launch_any<kGk>(w, gwk, gk, 0.f, B, C, T, as_stream(stream), "timex_backward(gk)");
}

extern "C" int rwkvb200_timex_backward_reduced(const float* w, const float* k, const float* gwk, float* gw_sum,
                                               float* gk, int B, int C, int T, void* stream) {
    if (int e = check_dims(B, C, T, "timex_backward_reduced")) return e;
    RWKV_NOTNULL(w); RWKV_NOTNULL(k); RWKV_NOTNULL(gwk); RWKV_NOTNULL(gw_sum); RWKV_NOTNULL(gk);
    // The per-row filter gradients go into the gk buffer (same shape, written afterwards), are summed over the
    // batch in a fixed order, and only then gk is computed: no extra memory, and the sum does not depend on the
    // order in which thread blocks run (an atomic sum over the batch groups was 3 % faster and did).
    if (int e = launch_any<kGw>(gwk, k, gk, 0.f, B, C, T, as_stream(stream), "timex_backward_reduced(gw)")) return e;
    if (int e = rwkvb200_reduce_batch_partials(RWKVB200_F32, B, C * T, gk, gw_sum, stream)) return e;
    return launch_any<kGk>(w, gwk, gk, 0.f, B, C, T, as_stream(stream), "timex_backward_reduced(gk)");
}
