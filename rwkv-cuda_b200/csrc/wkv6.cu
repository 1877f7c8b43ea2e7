// RWKV-6 WKV (per-token, per-channel decay), with optional initial / final state.
// fp32 or bf16 activations, fp32 state and accumulation.
//
// Operator (wkv6/run.py:183-218, wkv6_state/run.py:137-165 of the reference project), per (b,h):
//   y_t[i] = sum_j r_t[j] ( u[j] k_t[j] v_t[i] + S[i,j] ),   S[i,j] <- d_t[j] S[i,j] + k_t[j] v_t[i]
//   d_t = exp(-exp(w_raw_t));  S_0 = s0 (value i, key j) or zero.
// Serves three reference operators through one kernel pair:
//   wkv6       decay input is w = -exp(w_raw) in fp32 (the harness's pre-op), no state
//   wkv6state  decay input is w_raw in the activation dtype, state s / gs in the activation dtype
//   *_ex       as wkv6state with fp32 s0, final state sT out and its gradient dsT in
//
// One CTA per (batch, head), thread x owns one line of the N x N state in registers; vectors
// are exchanged through a double-buffered shared-memory stage, one barrier per token, with
// the next token's elements prefetched into registers.
//
// Backward: sweep 1 (forward in time, thread = key i) rebuilds S[:,i] and emits gr, gu and
// P_t[i] = r_t[i] sum_j gy_t[j] S_t[j,i] into an fp32 scratch (B,T,C).  Sweep 2 (reverse)
// carries D = dL/dS both by key line (gk, gw, ds0) and by value line (gv).  The decay gradient
// uses  A_t = sum_j D_{t-1}[j,i] S_t[j,i]:  with Q_t[i] = k_t[i] sum_j D_t[j,i] v_t[j]
//   dL/dlog d_t[i] = A_{t+1} - Q_t,     A_t = A_{t+1} - Q_t + P_t,    A_T = sum_j dsT[j,i] S_T[j,i]
// so no per-thread history of states is kept (the reference keeps T*N floats per thread and
// fails beyond T = 64..128) and T is unlimited.
#include <atomic>
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

enum StateKind { kNone = 0, kElem = 1, kF32 = 2 };

template <typename E>
__device__ __forceinline__ float load_state(const void* p, int kind, i64 idx) {
    if (kind == kF32) return reinterpret_cast<const float*>(p)[idx];
    if (kind == kElem) return to_f(reinterpret_cast<const E*>(p)[idx]);
    return 0.f;
}
template <typename E>
__device__ __forceinline__ void store_state(void* p, int kind, i64 idx, float x) {
    if (kind == kF32) reinterpret_cast<float*>(p)[idx] = x;
    else if (kind == kElem) reinterpret_cast<E*>(p)[idx] = from_f<E>(x);
}

// decay and d(log decay)/d(w_raw) from the stored decay input
template <typename E>
__device__ __forceinline__ void decay_of(const void* w, bool raw, i64 idx, float& d, float& dlog) {
    if (raw) {
        const float e = expf(to_f(reinterpret_cast<const E*>(w)[idx]));
        dlog = -e;
        d = expf(-e);
    } else {
        dlog = reinterpret_cast<const float*>(w)[idx];
        d = expf(dlog);
    }
}

// ------------------------------------------------------------------------------------
template <typename E, int NMAX>
__global__ void __launch_bounds__(NMAX) wkv6_forward_kernel(int T, int C, int H, int N, const E* __restrict__ r_,
                                                           const E* __restrict__ k_, const E* __restrict__ v_,
                                                           const void* __restrict__ w_, int w_raw,
                                                           const E* __restrict__ u_, const void* __restrict__ s0_,
                                                           int s0_kind, E* __restrict__ y_, float* __restrict__ sT_,
                                                           const int* __restrict__ only_if_) {
    if (only_if_ != nullptr && only_if_[blockIdx.x & (kChunkedFlagUnits - 1)] == 0) return;   // fallback launch: the chunked kernel's result stands for this unit
    const int b = blockIdx.x / H, h = blockIdx.x - b * H, i = threadIdx.x;
    const bool live = i < N;
    __shared__ Stage<NMAX> rs, ks, ds;
    __shared__ __align__(16) float us[NMAX];
    us[i] = live ? to_f(u_[h * N + i]) : 0.f;

    const i64 sbase = ((i64)(b * H + h) * N + i) * N;  // row i of the state: [value i][key j]
    float S[NMAX];
#pragma unroll
    for (int j = 0; j < NMAX; ++j) S[j] = (live && j < N) ? load_state<E>(s0_, s0_kind, sbase + j) : 0.f;

    const i64 base = (i64)b * T * C + h * N + i;
    float rn = 0.f, kn = 0.f, vn = 0.f, dn = 0.f, dl;
    if (live) {
        rn = to_f(r_[base]); kn = to_f(k_[base]); vn = to_f(v_[base]);
        decay_of<E>(w_, w_raw, base, dn, dl);
    }
    for (int t = 0; t < T; ++t) {
        const int p = t & 1;
        rs.a[p][i] = rn; ks.a[p][i] = kn; ds.a[p][i] = dn;
        const float v = vn;
        __syncthreads();
        if (t + 1 < T && live) {
            const i64 o = base + (i64)(t + 1) * C;
            rn = to_f(r_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]);
            decay_of<E>(w_, w_raw, o, dn, dl);
        }
        float y = 0.f;
#pragma unroll
        for (int j = 0; j < NMAX; j += 4) {
            const float4 r4 = *reinterpret_cast<const float4*>(&rs.a[p][j]);
            const float4 k4 = *reinterpret_cast<const float4*>(&ks.a[p][j]);
            const float4 d4 = *reinterpret_cast<const float4*>(&ds.a[p][j]);
            const float4 u4 = *reinterpret_cast<const float4*>(&us[j]);
            const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
            const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x = kk[e] * v;
                y = fmaf(rr[e], fmaf(uu[e], x, S[j + e]), y);
                S[j + e] = fmaf(S[j + e], dd[e], x);
            }
        }
        if (live) y_[base + (i64)t * C] = from_f<E>(y);
    }
    if (sT_ != nullptr && live) {
#pragma unroll
        for (int j = 0; j < NMAX; ++j)
            if (j < N) sT_[sbase + j] = S[j];
    }
}

// ------------------------------------------------------------------------------------
template <typename E, int NMAX>
__global__ void __launch_bounds__(NMAX) wkv6_backward_kernel(
    int T, int C, int H, int N, const E* __restrict__ r_, const E* __restrict__ k_, const E* __restrict__ v_,
    const void* __restrict__ w_, int w_raw, const E* __restrict__ u_, const void* __restrict__ s0_, int s0_kind,
    const E* __restrict__ gy_, const float* __restrict__ dsT_, E* __restrict__ gr_, E* __restrict__ gk_,
    E* __restrict__ gv_, E* __restrict__ gw_, E* __restrict__ gu_, void* __restrict__ ds0_, int ds0_kind,
    float* __restrict__ scratch_, const int* __restrict__ only_if_) {
    if (only_if_ != nullptr && only_if_[blockIdx.x & (kChunkedFlagUnits - 1)] == 0) return;   // fallback launch: the chunked kernels' result stands for this unit
    const int b = blockIdx.x / H, h = blockIdx.x - b * H, i = threadIdx.x;
    const bool live = i < N;
    __shared__ Stage<NMAX> rs, ks, vs, gs, ds;
    __shared__ __align__(16) float us[NMAX];
    us[i] = live ? to_f(u_[h * N + i]) : 0.f;
    __syncthreads();
    const float u = us[i];
    const i64 base = (i64)b * T * C + h * N + i;
    const i64 sbase = (i64)(b * H + h) * N * N;  // state block [value][key]

    float S[NMAX], D2[NMAX];
    float A = 0.f;

    // ---- sweep 1 (forward): thread = key i, S[j] = S[value j][key i] -------------------
    {
#pragma unroll
        for (int j = 0; j < NMAX; ++j)
            S[j] = (live && j < N) ? load_state<E>(s0_, s0_kind, sbase + (i64)j * N + i) : 0.f;
        float gu = 0.f;
        float rn = 0.f, kn = 0.f, vn = 0.f, gn = 0.f, dn = 0.f, dl;
        if (live) {
            rn = to_f(r_[base]); kn = to_f(k_[base]); vn = to_f(v_[base]); gn = to_f(gy_[base]);
            decay_of<E>(w_, w_raw, base, dn, dl);
        }
        for (int t = 0; t < T; ++t) {
            const int p = t & 1;
            vs.a[p][i] = vn; gs.a[p][i] = gn;
            const float r = rn, k = kn, d = dn;
            __syncthreads();
            if (t + 1 < T && live) {
                const i64 o = base + (i64)(t + 1) * C;
                rn = to_f(r_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]); gn = to_f(gy_[o]);
                decay_of<E>(w_, w_raw, o, dn, dl);
            }
            float sg = 0.f, vg = 0.f;
#pragma unroll
            for (int j = 0; j < NMAX; ++j) {
                const float vv = vs.a[p][j], g = gs.a[p][j];
                sg = fmaf(S[j], g, sg);
                vg = fmaf(vv, g, vg);
                S[j] = fmaf(S[j], d, k * vv);
            }
            if (live) {
                gr_[base + (i64)t * C] = from_f<E>(fmaf(u * k, vg, sg));
                scratch_[base + (i64)t * C] = r * sg;
            }
            gu = fmaf(r * k, vg, gu);
        }
        if (live) gu_[(i64)b * C + h * N + i] = from_f<E>(gu);
        if (dsT_ != nullptr && live) {
#pragma unroll
            for (int j = 0; j < NMAX; ++j)
                if (j < N) A = fmaf(dsT_[sbase + (i64)j * N + i], S[j], A);
        }
    }

    // ---- sweep 2 (reverse): S becomes D[value j][key i]; D2[j] = D[value i][key j] ------
    {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < NMAX; ++j) {
            const bool in = live && j < N && dsT_ != nullptr;
            S[j] = in ? dsT_[sbase + (i64)j * N + i] : 0.f;
            D2[j] = in ? dsT_[sbase + (i64)i * N + j] : 0.f;
        }
        const i64 last = base + (i64)(T - 1) * C;
        float rn = 0.f, kn = 0.f, vn = 0.f, gn = 0.f, dn = 0.f, dl = 0.f, pn = 0.f;
        if (live) {
            rn = to_f(r_[last]); kn = to_f(k_[last]); vn = to_f(v_[last]); gn = to_f(gy_[last]);
            decay_of<E>(w_, w_raw, last, dn, dl);
            pn = scratch_[last];
        }
        for (int t = T - 1; t >= 0; --t) {
            const int p = t & 1;
            rs.a[p][i] = rn; ks.a[p][i] = kn; vs.a[p][i] = vn; gs.a[p][i] = gn; ds.a[p][i] = dn;
            const float r = rn, k = kn, g = gn, d = dn, dlog = dl, P = pn;
            __syncthreads();
            if (t > 0 && live) {
                const i64 o = base + (i64)(t - 1) * C;
                rn = to_f(r_[o]); kn = to_f(k_[o]); vn = to_f(v_[o]); gn = to_f(gy_[o]);
                decay_of<E>(w_, w_raw, o, dn, dl);
                pn = scratch_[o];
            }
            float dv = 0.f, gyv = 0.f, gv = 0.f;
#pragma unroll
            for (int j = 0; j < NMAX; ++j) {
                const float vv = vs.a[p][j], gg = gs.a[p][j], rr = rs.a[p][j];
                dv = fmaf(S[j], vv, dv);
                gyv = fmaf(gg, vv, gyv);
                S[j] = fmaf(S[j], d, r * gg);
                const float x2 = g * rr;
                gv = fmaf(fmaf(us[j], x2, D2[j]), ks.a[p][j], gv);
                D2[j] = fmaf(D2[j], ds.a[p][j], x2);
            }
            const float Q = k * dv;
            if (live) {
                const i64 o = base + (i64)t * C;
                gk_[o] = from_f<E>(fmaf(u * r, gyv, dv));
                gv_[o] = from_f<E>(gv);
                gw_[o] = from_f<E>((A - Q) * dlog);
            }
            A = A - Q + P;
        }
        if (ds0_kind != kNone && live) {
#pragma unroll
            for (int j = 0; j < NMAX; ++j)
                if (j < N) store_state<E>(ds0_, ds0_kind, sbase + (i64)j * N + i, S[j]);
        }
    }
}

static int g_wkv6_chunked_enabled = 1;

template <typename E>
bool chunked_ok(int T, int N, std::initializer_list<const void*> ps) {
    if (!g_wkv6_chunked_enabled || !std::is_same<E, bf16>::value || N != 64 || T % 16 != 0) return false;
    for (const void* p : ps)
        if (p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) != 0) return false;
    return true;
}

template <typename E>
int launch_fwd(int B, int T, int C, int H, const void* r, const void* k, const void* v, const void* w, int w_raw,
               const void* u, const void* s0, int s0_kind, void* y, float* sT, cudaStream_t st, const char* what) {
    const int N = C / H;
    const int* only_if = nullptr;
    if (chunked_ok<E>(T, N, {r, k, v, w, u, s0, y, sT})) {
        // tensor-core kernel first; the general-shape kernel below then only runs if that one found a
        // chunk whose decay is too strong for the chunked form
        int* flag = wkv6_chunked_flag(st);   // NULL: every slot is taken, the general-shape kernel runs alone
        if (flag != nullptr) {
            RWKV_REQUIRE(cudaMemsetAsync(flag, 0, sizeof(int) * kChunkedFlagUnits, st) == cudaSuccess, RWKVB200_ECUDA, "%s: clearing the device flag failed", what);
            if (int e = wkv6_chunked_forward(B, T, H, r, k, v, w, w_raw, u, s0, s0_kind, y, sT, nullptr, flag, st)) return e;
            only_if = flag;
        }
    }
#define RWKV_GO(NM)                                                                                              \
    wkv6_forward_kernel<E, NM><<<B * H, NM, 0, st>>>(T, C, H, N, (const E*)r, (const E*)k, (const E*)v, w, w_raw, \
                                                      (const E*)u, s0, s0_kind, (E*)y, sT, only_if)
    switch (head_capacity(N)) {
        case 32: RWKV_GO(32); break;
        case 64: RWKV_GO(64); break;
        default: RWKV_GO(128); break;
    }
#undef RWKV_GO
    return check_launch(what);
}

template <typename E>
int launch_bwd(int B, int T, int C, int H, const void* r, const void* k, const void* v, const void* w, int w_raw,
               const void* u, const void* s0, int s0_kind, const void* gy, const float* dsT, void* gr, void* gk,
               void* gv, void* gw, void* gu, void* ds0, int ds0_kind, void* scratch, cudaStream_t st,
               const char* what, bool big_scratch = true) {
    const int N = C / H;
    const int* only_if = nullptr;
    if (big_scratch && chunked_ok<E>(T, N, {r, k, v, w, u, s0, gy, dsT, gr, gk, gv, gw, gu, ds0, scratch})) {
        // tensor-core kernels first: a forward pass that leaves the chunk-start states in the scratch
        // buffer, then the reverse pass; the general-shape kernel below then only runs if a chunk's decay
        // was too strong for the chunked form (it reuses the front of the same scratch buffer)
        int* flag = wkv6_chunked_flag(st);   // NULL: every slot is taken, the general-shape kernel runs alone
        if (flag != nullptr) {
            RWKV_REQUIRE(cudaMemsetAsync(flag, 0, sizeof(int) * kChunkedFlagUnits, st) == cudaSuccess, RWKVB200_ECUDA, "%s: clearing the device flag failed", what);
            float* ck = static_cast<float*>(scratch);
            if (int e = wkv6_backward_with_states(B, T, H, r, k, v, w, w_raw, u, s0, s0_kind, gy, dsT, ck, gr, gk, gv, gw, gu, ds0,
                                                  ds0_kind, flag, st))
                return e;
            only_if = flag;
        }
    }
#define RWKV_GO(NM)                                                                                               \
    wkv6_backward_kernel<E, NM><<<B * H, NM, 0, st>>>(T, C, H, N, (const E*)r, (const E*)k, (const E*)v, w, w_raw, \
                                                       (const E*)u, s0, s0_kind, (const E*)gy, dsT, (E*)gr,       \
                                                       (E*)gk, (E*)gv, (E*)gw, (E*)gu, ds0, ds0_kind,             \
                                                       (float*)scratch, only_if)
    switch (head_capacity(N)) {
        case 32: RWKV_GO(32); break;
        case 64: RWKV_GO(64); break;
        default: RWKV_GO(128); break;
    }
#undef RWKV_GO
    return check_launch(what);
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

extern "C" size_t rwkvb200_wkv6_scratch_bytes(int B, int T, int C) {
    if (B <= 0 || T <= 0 || C <= 0) return 0;
    // 16 bytes per element: the chunked backward (bf16, head size 64, T a multiple of 16) keeps one
    // fp32 64x64 state per 16 tokens and head here; the general-shape backward uses the first quarter
    return (size_t)B * T * C * sizeof(float) * 4;
}

extern "C" int rwkvb200_wkv6_forward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                     const void* v, const float* w, const void* u, void* y, void* stream) {
    if (int e = check_dims("wkv6_forward", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(y);
    return dtype == RWKVB200_F32
               ? launch_fwd<float>(B, T, C, H, r, k, v, w, 0, u, nullptr, kNone, y, nullptr, as_stream(stream), "wkv6_forward")
               : launch_fwd<bf16>(B, T, C, H, r, k, v, w, 0, u, nullptr, kNone, y, nullptr, as_stream(stream), "wkv6_forward");
}

extern "C" int rwkvb200_wkv6_backward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                      const void* v, const float* w, const void* u, const void* gy, void* gr,
                                      void* gk, void* gv, void* gw, void* gu, void* scratch, void* stream) {
    if (int e = check_dims("wkv6_backward", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(gy);
    RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu); RWKV_NOTNULL(scratch);
    return dtype == RWKVB200_F32
               ? launch_bwd<float>(B, T, C, H, r, k, v, w, 0, u, nullptr, kNone, gy, nullptr, gr, gk, gv, gw, gu,
                                   nullptr, kNone, scratch, as_stream(stream), "wkv6_backward")
               : launch_bwd<bf16>(B, T, C, H, r, k, v, w, 0, u, nullptr, kNone, gy, nullptr, gr, gk, gv, gw, gu,
                                  nullptr, kNone, scratch, as_stream(stream), "wkv6_backward");
}

// ---- backward without a scratch argument ---------------------------------------------------
// Some callers of this library are not allowed to allocate device memory at the point where
// they run the backward: a latency-critical host thread that must never enter the device
// allocator, an embedding runtime that owns all device memory and hands out fixed buffers only,
// a process whose memory pool is already fully committed.  For them the P_t buffer lives in a
// fixed array that is part of the loaded library image (every GPU that loads the library keeps
// these 32 MiB until the process exits).
namespace rwkvb200 {
namespace {
constexpr size_t kNoAllocMaxElems = size_t(8) << 20;  // B*T*C limit: 8 Mi floats = 32 MiB
static __device__ __align__(256) float g_wkv6_noalloc_scratch[kNoAllocMaxElems];
constexpr int kMaxDevices = 64;
std::atomic<float*> g_noalloc_ptr[kMaxDevices] = {};  // device address of the array, per device, filled on first use
}  // namespace
}  // namespace rwkvb200

extern "C" size_t rwkvb200_wkv6_backward_noalloc_max_elems(void) { return kNoAllocMaxElems; }

extern "C" int rwkvb200_wkv6_backward_noalloc(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                              const void* v, const float* w, const void* u, const void* gy,
                                              void* gr, void* gk, void* gv, void* gw, void* gu, void* stream) {
    if (int e = check_dims("wkv6_backward_noalloc", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(gy);
    RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu);
    const size_t need = (size_t)B * T * C;
    RWKV_REQUIRE(need <= kNoAllocMaxElems, RWKVB200_EINVAL,
                 "wkv6_backward_noalloc: B*T*C = %zu exceeds the built-in scratch of %zu elements; "
                 "use rwkvb200_wkv6_backward with a caller-provided scratch buffer",
                 need, kNoAllocMaxElems);
    int dev = -1;
    cudaError_t ce = cudaGetDevice(&dev);
    RWKV_REQUIRE(ce == cudaSuccess && dev >= 0 && dev < kMaxDevices, RWKVB200_ECUDA,
                 "wkv6_backward_noalloc: cudaGetDevice: %s (device %d)", cudaGetErrorString(ce), dev);
    float* scratch = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        // In host code the array's name is only a handle; the device address has to be asked for,
        // once per device, with that device current.
        void* p = nullptr;
        ce = cudaGetSymbolAddress(&p, g_wkv6_noalloc_scratch);
        RWKV_REQUIRE(ce == cudaSuccess && p != nullptr, RWKVB200_ECUDA,
                     "wkv6_backward_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(ce));
        scratch = static_cast<float*>(p);
        g_noalloc_ptr[dev].store(scratch, std::memory_order_release);
    }
    // The kernel writes every scratch element it later reads (same thread, same launch), so
    // nothing has to be cleared between calls.
    return dtype == RWKVB200_F32
               ? launch_bwd<float>(B, T, C, H, r, k, v, w, 0, u, nullptr, kNone, gy, nullptr, gr, gk, gv, gw, gu,
                                   nullptr, kNone, scratch, as_stream(stream), "wkv6_backward_noalloc", false)
               : launch_bwd<bf16>(B, T, C, H, r, k, v, w, 0, u, nullptr, kNone, gy, nullptr, gr, gk, gv, gw, gu,
                                  nullptr, kNone, scratch, as_stream(stream), "wkv6_backward_noalloc", false);
}

extern "C" int rwkvb200_wkv6state_forward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                          const void* v, const void* w, const void* u, const void* s, void* y,
                                          void* stream) {
    if (int e = check_dims("wkv6state_forward", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(s); RWKV_NOTNULL(y);
    return dtype == RWKVB200_F32
               ? launch_fwd<float>(B, T, C, H, r, k, v, w, 1, u, s, kElem, y, nullptr, as_stream(stream), "wkv6state_forward")
               : launch_fwd<bf16>(B, T, C, H, r, k, v, w, 1, u, s, kElem, y, nullptr, as_stream(stream), "wkv6state_forward");
}

extern "C" int rwkvb200_wkv6state_backward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                           const void* v, const void* w, const void* u, const void* s,
                                           const void* gy, void* gr, void* gk, void* gv, void* gw, void* gu,
                                           void* gs, void* scratch, void* stream) {
    if (int e = check_dims("wkv6state_backward", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(s);
    RWKV_NOTNULL(gy); RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu);
    RWKV_NOTNULL(gs); RWKV_NOTNULL(scratch);
    return dtype == RWKVB200_F32
               ? launch_bwd<float>(B, T, C, H, r, k, v, w, 1, u, s, kElem, gy, nullptr, gr, gk, gv, gw, gu, gs, kElem,
                                   scratch, as_stream(stream), "wkv6state_backward")
               : launch_bwd<bf16>(B, T, C, H, r, k, v, w, 1, u, s, kElem, gy, nullptr, gr, gk, gv, gw, gu, gs, kElem,
                                  scratch, as_stream(stream), "wkv6state_backward");
}

extern "C" int rwkvb200_wkv6state_forward_ex(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                             const void* v, const void* w, const void* u, const float* s0, void* y,
                                             float* sT, void* stream) {
    if (int e = check_dims("wkv6state_forward_ex", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(y);
    const int sk = s0 ? kF32 : kNone;
    return dtype == RWKVB200_F32
               ? launch_fwd<float>(B, T, C, H, r, k, v, w, 1, u, s0, sk, y, sT, as_stream(stream), "wkv6state_forward_ex")
               : launch_fwd<bf16>(B, T, C, H, r, k, v, w, 1, u, s0, sk, y, sT, as_stream(stream), "wkv6state_forward_ex");
}

// Kernels of the bf16 / head-size-64 forward and backward of RWKV-5 and RWKV-6: 1 (default) = tcgen05, 32-token chunks
// (wkv6_l32_fwd.cu, wkv6_l32_bwd.cu); 0 = mma.sync, 16-token chunks (wkv6_chunked.cu).  For tests and measurements.
extern "C" int rwkvb200_wkv6_select_forward(int kernel) {
    RWKV_REQUIRE(kernel == 0 || kernel == 1, RWKVB200_EINVAL, "wkv6_select_forward: kernel %d not in 0..1", kernel);
    wkv6_select_forward(kernel);
    wkv6_select_backward(kernel);
    return RWKVB200_OK;
}

// The forward split over time (wkv6_tsplit.cu): `segments` pieces of T/segments tokens run at the same time.
// Tensor-core shapes only (bf16, head size 64, T/segments a multiple of 16, 16-byte aligned tensors); a decay too
// strong for the chunked form makes the general-shape kernel redo the whole call, as in the unsplit forward.
extern "C" size_t rwkvb200_wkv6_tsplit_bytes(int B, int T, int C, int H, int segments) {
    (void)T;
    return (B > 0 && C > 0 && H > 0 && segments > 0) ? wkv6_tsplit_bytes(B, C, H, segments) : 0;
}

extern "C" int rwkvb200_wkv6state_forward_tsplit(int dtype, int B, int T, int C, int H, int segments, const void* r,
                                                 const void* k, const void* v, const void* w, const void* u,
                                                 const float* s0, void* y, float* sT, void* work, void* stream) {
    if (int e = check_dims("wkv6state_forward_tsplit", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(y); RWKV_NOTNULL(work);
    const int K = segments, N = C / H;
    RWKV_REQUIRE(K >= 1 && T % K == 0 && (T / K) % 16 == 0, RWKVB200_EINVAL,
                 "wkv6state_forward_tsplit: T = %d is not %d segments of a multiple of 16 tokens", T, K);
    RWKV_REQUIRE(dtype == RWKVB200_BF16 && chunked_ok<bf16>(T / K, N, {r, k, v, w, u, s0, y, sT, work}), RWKVB200_EINVAL,
                 "wkv6state_forward_tsplit: needs bf16 tensors, head size 64, 16-byte alignment");
    cudaStream_t st = as_stream(stream);
    int* flag = wkv6_chunked_flag(st);
    if (flag == nullptr || K == 1)   // no flag word left for this stream, or nothing to split: the plain forward
        return launch_fwd<bf16>(B, T, C, H, r, k, v, w, 1, u, s0, s0 ? kF32 : kNone, y, sT, st, "wkv6state_forward_tsplit");
    RWKV_REQUIRE(cudaMemsetAsync(flag, 0, sizeof(int) * kChunkedFlagUnits, st) == cudaSuccess, RWKVB200_ECUDA,
                 "wkv6state_forward_tsplit: clearing the device flag failed");
    float* wk = static_cast<float*>(work);
    float* start = wk + (size_t)B * K * H * N * N;
    // 1. every segment from a zero state, states only  2. segment start states  3. every segment with its start state
    if (int e = wkv6_chunked_forward(B * K, T / K, H, r, k, v, w, 1, u, nullptr, kNone, nullptr, wk, nullptr, flag, st, K)) return e;
    if (int e = wkv6_tsplit_states(B, T, C, H, K, w, 1, s0, wk, sT, st)) return e;
    if (int e = wkv6_chunked_forward(B * K, T / K, H, r, k, v, w, 1, u, start, kF32, y, nullptr, nullptr, flag, st, K)) return e;
    // a chunk whose decay is too strong for the chunked form: the general-shape kernel redoes the call
    wkv6_forward_kernel<bf16, 64><<<B * H, 64, 0, st>>>(T, C, H, N, (const bf16*)r, (const bf16*)k, (const bf16*)v, w, 1,
                                                       (const bf16*)u, s0, s0 ? kF32 : kNone, (bf16*)y, sT, flag);
    return check_launch("wkv6state_forward_tsplit");
}

// Training flow with saved states: the forward leaves the states at the start of every 32-token chunk (and the
// "decay too strong" flags of its units) in `saved`, a buffer of rwkvb200_wkv6_scratch_bytes(B,T,C) bytes, and the
// backward uses them instead of running its own pass over the sequence to rebuild them.  The forward returns
// RWKVB200_OK when it saved them and 1 when it ran on kernels that do not (other dtype, head size, alignment, no
// tensor maps, no flag words left): pass that as `saved_valid` = 0 to the backward, which then behaves as
// rwkvb200_wkv6state_backward_ex with `saved` as its scratch.  No counterpart in the reference.
extern "C" int rwkvb200_wkv6state_forward_saved(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                                const void* v, const void* w, const void* u, const float* s0, void* y,
                                                float* sT, void* saved, void* stream) {
    if (int e = check_dims("wkv6state_forward_saved", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(y); RWKV_NOTNULL(saved);
    const int N = C / H, sk = s0 ? kF32 : kNone;
    cudaStream_t st = as_stream(stream);
    int* flag = nullptr;
    if (dtype == RWKVB200_BF16 && wkv6_forward_choice() && chunked_ok<bf16>(T, N, {r, k, v, w, u, s0, y, sT, saved}))
        flag = wkv6_chunked_flag(st);
    if (flag != nullptr) {
        RWKV_REQUIRE(cudaMemsetAsync(flag, 0, sizeof(int) * kChunkedFlagUnits, st) == cudaSuccess, RWKVB200_ECUDA,
                     "wkv6state_forward_saved: clearing the device flags failed");
        const int rc = wkv6_l32_forward(B, T, H, r, k, v, w, 1, u, s0, sk, y, sT, static_cast<float*>(saved), flag, st, 1);
        if (rc < 0) return rc;
        if (rc == 0) {
            // flagged units: the general-shape kernel redoes them; the flags travel with the saved states
            wkv6_forward_kernel<bf16, 64><<<B * H, 64, 0, st>>>(T, C, H, N, (const bf16*)r, (const bf16*)k, (const bf16*)v, w, 1,
                                                               (const bf16*)u, s0, sk, (bf16*)y, sT, flag);
            if (int e = check_launch("wkv6state_forward_saved")) return e;
            char* tail = static_cast<char*>(saved) + rwkvb200_wkv6_scratch_bytes(B, T, C) - sizeof(int) * kChunkedFlagUnits;
            RWKV_REQUIRE(cudaMemcpyAsync(tail, flag, sizeof(int) * kChunkedFlagUnits, cudaMemcpyDeviceToDevice, st) == cudaSuccess,
                         RWKVB200_ECUDA, "wkv6state_forward_saved: saving the device flags failed");
            return RWKVB200_OK;
        }
    }
    const int e = dtype == RWKVB200_F32
                      ? launch_fwd<float>(B, T, C, H, r, k, v, w, 1, u, s0, sk, y, sT, st, "wkv6state_forward_saved")
                      : launch_fwd<bf16>(B, T, C, H, r, k, v, w, 1, u, s0, sk, y, sT, st, "wkv6state_forward_saved");
    return e ? e : 1;
}

extern "C" int rwkvb200_wkv6state_backward_saved(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                                 const void* v, const void* w, const void* u, const float* s0,
                                                 const void* gy, const float* dsT, void* gr, void* gk, void* gv,
                                                 void* gw, void* gu, float* ds0, void* saved, int saved_valid, void* stream) {
    if (int e = check_dims("wkv6state_backward_saved", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(gy);
    RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu); RWKV_NOTNULL(saved);
    const int N = C / H, sk = s0 ? kF32 : kNone, dk = ds0 ? kF32 : kNone;
    cudaStream_t st = as_stream(stream);
    int* flag = nullptr;
    if (saved_valid && dtype == RWKVB200_BF16 && chunked_ok<bf16>(T, N, {r, k, v, w, u, s0, gy, dsT, gr, gk, gv, gw, gu, ds0, saved}))
        flag = wkv6_chunked_flag(st);
    if (flag != nullptr) {
        const char* tail = static_cast<const char*>(saved) + rwkvb200_wkv6_scratch_bytes(B, T, C) - sizeof(int) * kChunkedFlagUnits;
        RWKV_REQUIRE(cudaMemcpyAsync(flag, tail, sizeof(int) * kChunkedFlagUnits, cudaMemcpyDeviceToDevice, st) == cudaSuccess,
                     RWKVB200_ECUDA, "wkv6state_backward_saved: restoring the device flags failed");
        if (int e = wkv6_l32_backward(B, T, H, r, k, v, w, 1, u, gy, dsT, static_cast<const float*>(saved), gr, gk, gv, gw, gu, ds0, dk, st))
            return e;
        // flagged units: the general-shape kernel redoes them (it uses the front of `saved` as its scratch, after
        // the kernel above has read the states)
        wkv6_backward_kernel<bf16, 64><<<B * H, 64, 0, st>>>(T, C, H, N, (const bf16*)r, (const bf16*)k, (const bf16*)v, w, 1,
                                                            (const bf16*)u, s0, sk, (const bf16*)gy, dsT, (bf16*)gr, (bf16*)gk,
                                                            (bf16*)gv, (bf16*)gw, (bf16*)gu, ds0, dk, static_cast<float*>(saved), flag);
        return check_launch("wkv6state_backward_saved");
    }
    return dtype == RWKVB200_F32
               ? launch_bwd<float>(B, T, C, H, r, k, v, w, 1, u, s0, sk, gy, dsT, gr, gk, gv, gw, gu, ds0, dk, saved, st, "wkv6state_backward_saved")
               : launch_bwd<bf16>(B, T, C, H, r, k, v, w, 1, u, s0, sk, gy, dsT, gr, gk, gv, gw, gu, ds0, dk, saved, st, "wkv6state_backward_saved");
}

extern "C" int rwkvb200_wkv6state_backward_ex(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                              const void* v, const void* w, const void* u, const float* s0,
                                              const void* gy, const float* dsT, void* gr, void* gk, void* gv,
                                              void* gw, void* gu, float* ds0, void* scratch, void* stream) {
    if (int e = check_dims("wkv6state_backward_ex", dtype, B, T, C, H)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(w); RWKV_NOTNULL(u); RWKV_NOTNULL(gy);
    RWKV_NOTNULL(gr); RWKV_NOTNULL(gk); RWKV_NOTNULL(gv); RWKV_NOTNULL(gw); RWKV_NOTNULL(gu); RWKV_NOTNULL(scratch);
    const int sk = s0 ? kF32 : kNone, dk = ds0 ? kF32 : kNone;
    return dtype == RWKVB200_F32
               ? launch_bwd<float>(B, T, C, H, r, k, v, w, 1, u, s0, sk, gy, dsT, gr, gk, gv, gw, gu, ds0, dk, scratch,
                                   as_stream(stream), "wkv6state_backward_ex")
               : launch_bwd<bf16>(B, T, C, H, r, k, v, w, 1, u, s0, sk, gy, dsT, gr, gk, gv, gw, gu, ds0, dk, scratch,
                                  as_stream(stream), "wkv6state_backward_ex");
}
