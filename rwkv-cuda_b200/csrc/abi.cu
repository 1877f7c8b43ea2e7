// Error plumbing, library identity and the RWKV-7 entry points (argument checks + dispatch
// between the general-shape kernels and the N = 64 tensor-core path).
#include "common.cuh"
#include "wkv7_dispatch.cuh"
#include "wkv6_chunked.cuh"
#include <atomic>
#include <initializer_list>

namespace rwkvb200 {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: kernel launch failed: %s", what, cudaGetErrorString(e));
        return RWKVB200_ECUDA;
    }
    return RWKVB200_OK;
}

}  // namespace rwkvb200

using namespace rwkvb200;

extern "C" const char* rwkvb200_strerror(int code) {
    switch (code) {
        case RWKVB200_OK: return "ok";
        case RWKVB200_EINVAL: return "invalid argument";
        case RWKVB200_ENULL: return "null pointer";
        case RWKVB200_EALIGN: return "misaligned pointer";
        case RWKVB200_EUNSUPPORTED: return "unsupported configuration";
        case RWKVB200_ECUDA: return "CUDA error";
        default: return "unknown error";
    }
}

extern "C" const char* rwkvb200_last_error(void) { return g_err; }
extern "C" int rwkvb200_version(void) { return 100; }
extern "C" int rwkvb200_built_for_sm(void) { return 100; }

// 0 = automatic (tensor-core kernels where the shape allows), 1 = general-shape kernels only,
// 2 = tensor-core kernels or an error.  Read once per call; forward and backward of one operator call
// must see the same value (the saved buffers differ between the two kernel families).
static std::atomic<int> g_wkv7_path{0};
static std::atomic<int> g_wkv7_test_expire{0};
static std::atomic<int> g_wkv7_bwd_form{0};   // 0 automatic, 1 one-group kernels, 2 staged forward / two-stage backward

static int sm_count() {
    constexpr int kMaxDevices = 64;
    static std::atomic<int> cache[kMaxDevices] = {};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    if ((n = cache[dev].load()) != 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cache[dev].store(n);
    return n;
}

extern "C" int rwkvb200_wkv7_select_form(int form) {
    RWKV_REQUIRE(form >= 0 && form <= 2, RWKVB200_EINVAL, "wkv7_select_form: form %d not in 0..2", form);
    g_wkv7_bwd_form.store(form);
    return RWKVB200_OK;
}

extern "C" int rwkvb200_wkv7_select_path(int path) {
    RWKV_REQUIRE(path >= 0 && path <= 2, RWKVB200_EINVAL, "wkv7_select_path: path %d not in 0..2", path);
    g_wkv7_path.store(path);
    return RWKVB200_OK;
}

static std::atomic<int> g_no_tensor_maps{0};
bool rwkvb200::tensor_maps_disabled() { return g_no_tensor_maps.load() != 0; }
extern "C" int rwkvb200_test_disable_tensor_maps(int on) {
    g_no_tensor_maps.store(on ? 1 : 0);
    return RWKVB200_OK;
}

extern "C" int rwkvb200_wkv7_test_expire_next_forward(void) {
    g_wkv7_test_expire.store(1);
    return RWKVB200_OK;
}

static bool aligned16(std::initializer_list<const void*> ps) {
    for (const void* p : ps)
        if (p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) != 0) return false;
    return true;
}

// Forward and backward must agree on the layout of the saved buffers, so the choice depends
// on (path, dtype, N, chunk_len) only; misaligned tensors on the tensor-core path are an error.
static int wkv7_use_tensor_path(const char* what, int dtype, int N, int chunk, bool* use) {
    const int path = g_wkv7_path.load();
    const bool shape_ok = dtype == RWKVB200_BF16 && N == 64 && chunk == 16;
    if (path == 2)
        RWKV_REQUIRE(shape_ok, RWKVB200_EUNSUPPORTED, "%s: tensor-core path needs bf16, N=64, chunk_len=16", what);
    *use = shape_ok && path != 1;
    return RWKVB200_OK;
}

static int wkv7_check(const char* what, int dtype, int B, int T, int H, int N, int chunk) {
    RWKV_REQUIRE(dtype == RWKVB200_F32 || dtype == RWKVB200_BF16, RWKVB200_EINVAL, "%s: unknown dtype %d", what, dtype);
    RWKV_REQUIRE(B > 0 && T > 0 && H > 0 && N > 0 && chunk > 0, RWKVB200_EINVAL,
                 "%s: B=%d T=%d H=%d N=%d chunk_len=%d must be positive", what, B, T, H, N, chunk);
    RWKV_REQUIRE(B <= 65535, RWKVB200_EINVAL, "%s: B=%d exceeds 65535", what, B);
    RWKV_REQUIRE(N <= RWKVB200_MAX_HEAD_SIZE, RWKVB200_EUNSUPPORTED, "%s: head size %d > %d", what, N,
                 RWKVB200_MAX_HEAD_SIZE);
    RWKV_REQUIRE(T % chunk == 0, RWKVB200_EINVAL, "%s: T=%d is not a multiple of chunk_len=%d", what, T, chunk);
    return RWKVB200_OK;
}

extern "C" int rwkvb200_device_status(void) {
    const int f = wkv7_l32_fwd_error(), g = wkv7_l32_bwd_error();
    if (f < 0 || g < 0) {
        set_error("device_status: reading the status words failed");
        return RWKVB200_ECUDA;
    }
    const int p = wkv7_l32_bwdp_error(0), q = wkv7_l32_fwdp_error(0), r6 = wkv6_l32_error(0), b6 = wkv6_l32_bwd_error(0);
    if (p < 0 || q < 0 || r6 < 0 || b6 < 0) {
        set_error("device_status: reading the status words failed");
        return RWKVB200_ECUDA;
    }
    if (f) return 10 + f;
    if (g) return 20 + g;
    if (p) return p;            // the two-stage backward records 30.. (front group) or 40.. (back group)
    if (q) return q + 20;       // the staged RWKV-7 forward 50.. / 55.. / 60..
    if (r6) return r6 + 40;     // the staged RWKV-6 / RWKV-5 forward 70.. / 75.. / 80..
    return b6 ? b6 + 90 : 0;    // the tcgen05 RWKV-6 / RWKV-5 backward 91..
}

extern "C" int rwkvb200_device_status_clear(void) {
    RWKV_REQUIRE(wkv7_l32_clear_errors() == 0 && wkv7_l32_bwdp_error(1) == 0 && wkv7_l32_fwdp_error(1) == 0 && wkv6_l32_error(1) == 0 && wkv6_l32_bwd_error(1) == 0, RWKVB200_ECUDA, "device_status_clear: writing the status words failed");
    return RWKVB200_OK;
}

extern "C" int rwkvb200_wkv7_forward(int dtype, int B, int T, int H, int N, int chunk_len, const float* s0,
                                     const void* r, const void* w, const void* k, const void* v, const void* a,
                                     const void* b, void* y, float* sT, float* s, float* sa, void* stream) {
    if (int e = wkv7_check("wkv7_forward", dtype, B, T, H, N, chunk_len)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(w); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(a); RWKV_NOTNULL(b);
    RWKV_NOTNULL(y);
    RWKV_REQUIRE((s == nullptr) == (sa == nullptr), RWKVB200_EINVAL,
                 "wkv7_forward: s and sa must be given together (or both NULL for inference)");
    bool tensor;
    if (int e = wkv7_use_tensor_path("wkv7_forward", dtype, N, chunk_len, &tensor)) return e;
    if (tensor) {
        RWKV_REQUIRE(aligned16({s0, r, w, k, v, a, b, y, sT, s, sa}), RWKVB200_EALIGN,
                     "wkv7_forward: the bf16 N=64 path needs 16-byte aligned tensors");
        const int form = g_wkv7_bwd_form.load(), expire = g_wkv7_test_expire.exchange(0);
        // the staged form (three warp groups on consecutive chunks, inputs by TMA) is the faster one at every size
        if (!expire && form != 1) {
            const int rc = wkv7_l32_forward_pipelined(B, T, H, s0, r, w, k, v, a, b, y, sT, s, as_stream(stream));
            if (rc != 1) return rc;   // 1: no tensor maps on this driver, use the one-group kernel
        }
        return wkv7_l32_forward(B, T, H, s0, r, w, k, v, a, b, y, sT, s, expire, as_stream(stream));
    }
    return wkv7_generic_forward(dtype, B, T, H, N, chunk_len, s0, r, w, k, v, a, b, y, sT, s, sa, as_stream(stream));
}

extern "C" int rwkvb200_wkv7_backward(int dtype, int B, int T, int H, int N, int chunk_len, const void* r,
                                      const void* w, const void* k, const void* v, const void* a, const void* b,
                                      const void* dy, const float* dsT, const float* s, const float* sa, float* ds0,
                                      void* dr, void* dw, void* dk, void* dv, void* da, void* db, void* stream) {
    if (int e = wkv7_check("wkv7_backward", dtype, B, T, H, N, chunk_len)) return e;
    RWKV_NOTNULL(r); RWKV_NOTNULL(w); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(a); RWKV_NOTNULL(b);
    RWKV_NOTNULL(dy); RWKV_NOTNULL(s); RWKV_NOTNULL(sa);
    RWKV_NOTNULL(dr); RWKV_NOTNULL(dw); RWKV_NOTNULL(dk); RWKV_NOTNULL(dv); RWKV_NOTNULL(da); RWKV_NOTNULL(db);
    bool tensor;
    if (int e = wkv7_use_tensor_path("wkv7_backward", dtype, N, chunk_len, &tensor)) return e;
    if (tensor) {
        RWKV_REQUIRE(aligned16({r, w, k, v, a, b, dy, dsT, s, sa, ds0, dr, dw, dk, dv, da, db}), RWKVB200_EALIGN,
                     "wkv7_backward: the bf16 N=64 path needs 16-byte aligned tensors");
        // at most one unit per SM: the time is one unit's chain of chunks, which the two-stage form (one thread
        // block per SM, two warp groups on consecutive chunks) nearly halves; with more units per SM two
        // independent one-group blocks per SM give more throughput
        const int form = g_wkv7_bwd_form.load();
        if (form == 2 || (form == 0 && (long long)B * H <= sm_count()))
            return wkv7_l32_backward_pipelined(B, T, H, r, w, k, v, a, b, dy, dsT, s, ds0, dr, dw, dk, dv, da, db, as_stream(stream));
        return wkv7_l32_backward(B, T, H, r, w, k, v, a, b, dy, dsT, s, ds0, dr, dw, dk, dv, da, db, as_stream(stream));
    }
    return wkv7_generic_backward(dtype, B, T, H, N, chunk_len, r, w, k, v, a, b, dy, dsT, s, sa, ds0, dr, dw, dk, dv,
                                 da, db, as_stream(stream));
}

// Inference-shaped entry: advance the recurrent state by T >= 1 tokens in place and return y; nothing is
// saved for a backward pass and T needs no alignment (T = 1 is one decoding step).
extern "C" int rwkvb200_wkv7_state_update(int dtype, int B, int T, int H, int N, float* state, const void* r,
                                          const void* w, const void* k, const void* v, const void* a, const void* b,
                                          void* y, void* stream) {
    if (int e = wkv7_check("wkv7_state_update", dtype, B, T, H, N, 1)) return e;
    RWKV_NOTNULL(state); RWKV_NOTNULL(r); RWKV_NOTNULL(w); RWKV_NOTNULL(k); RWKV_NOTNULL(v); RWKV_NOTNULL(a); RWKV_NOTNULL(b);
    RWKV_NOTNULL(y);
    // long aligned prompts in bf16 with head size 64 take the tensor-core forward, everything else
    // (decoding steps, odd lengths, other head sizes, fp32) the general-shape kernel
    const bool tensor = g_wkv7_path.load() != 1 && dtype == RWKVB200_BF16 && N == 64 && T % 16 == 0 && T >= 64 &&
                        aligned16({state, r, w, k, v, a, b, y});
    if (tensor) {
        if (g_wkv7_bwd_form.load() != 1) {
            const int rc = wkv7_l32_forward_pipelined(B, T, H, state, r, w, k, v, a, b, y, state, nullptr, as_stream(stream));
            if (rc != 1) return rc;   // 1: no tensor maps on this driver, use the one-group kernel
        }
        return wkv7_l32_forward(B, T, H, state, r, w, k, v, a, b, y, state, nullptr, 0, as_stream(stream));
    }
    return wkv7_generic_forward(dtype, B, T, H, N, T, state, r, w, k, v, a, b, y, state, nullptr, nullptr, as_stream(stream));
}
