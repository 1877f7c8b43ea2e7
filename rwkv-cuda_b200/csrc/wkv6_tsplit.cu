// Two-level scan over time for the diagonal-decay recurrences (RWKV-5, RWKV-6): the forward of a launch with
// few (batch, head) units is split into K segments of T/K tokens that run at the same time.
//
// The reference has this for RWKV-5's static decay only (wkv5_bf16/cuda/wkv5_cuda_v3.cu:12-30
// kernel_forward_accumulate_state, :32-95 kernel_forward<false/true>, host :97-128).  The transition of one
// token, S <- S diag(d_t) + v_t k_t^T, is diagonal in the key index for a per-token decay as well, so over a
// segment  S_end = S_start diag(D) + L  with D = prod_t d_t (per key channel) and L = the end state of the
// segment started from zero.  Three steps:
//   1. every segment from a zero state, states only (the states-only instance of the chunked forward kernel,
//      on the (B*K, T/K, C) view of the tensors): L;
//   2. this file: D per segment, then per (batch, head) the K start states by the recurrence above (K steps
//      of N*N multiply-adds), and the final state;
//   3. every segment again with its start state: y (the chunked forward kernel, same view).
// Pays when B*H is small against the number of SMs: step 1 costs about 40 % of a forward pass.
#include "wkv6_tsplit.cuh"

namespace rwkvb200 {
namespace {

// log2 of the decay of one (token, channel); decay forms as in the chunked kernels:
// 0 = fp32 log-decay (B,T,C), 1 = bf16 raw input (B,T,C) with log-decay = -exp(w), 2 = fp32 decay value (C),
// 3 = fp32 log-decay (C)
template <int mode>
__device__ __forceinline__ float log2_decay(const void* w, i64 tok_idx, int ch) {
    constexpr float kLog2e = 1.4426950408889634f;
    if (mode == 0) return reinterpret_cast<const float*>(w)[tok_idx] * kLog2e;
    if (mode == 1) return -__expf(__bfloat162float(reinterpret_cast<const bf16*>(w)[tok_idx])) * kLog2e;
    if (mode == 2) return __log2f(reinterpret_cast<const float*>(w)[ch]);
    return reinterpret_cast<const float*>(w)[ch] * kLog2e;
}

// Dp[slice][(b*K + k)*C + c] = sum over a slice of the segment's tokens of log2 d_t[c] (the slices are added up in
// a fixed order by segment_states_kernel: results do not depend on the order in which blocks run).
// grid (C/128, B*K, slices), block (128 channels, 8 token lanes): a thread takes every 8th token of its slice,
// the 8 partial sums meet in shared memory.
template <int mode>
__global__ void __launch_bounds__(1024) segment_decay_kernel(int Tseg, int C, const void* __restrict__ w, float* __restrict__ Dl) {
    __shared__ float part[8][128];
    const int c = blockIdx.x * 128 + threadIdx.x, seg = blockIdx.y;
    const int per = (Tseg + gridDim.z - 1) / gridDim.z, t0 = blockIdx.z * per, t1 = min(Tseg, t0 + per);
    float acc = 0.f;
    if (c < C) {
        if (mode >= 2) {
            if (threadIdx.y == 0) acc = log2_decay<mode>(w, 0, c) * (float)(t1 - t0);
        } else {
            const i64 base = (i64)seg * Tseg * C + c;
            for (int t = t0 + threadIdx.y; t < t1; t += 8) acc += log2_decay<mode>(w, base + (i64)t * C, c);
        }
    }
    part[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) sum += part[q][threadIdx.x];
        Dl[((i64)blockIdx.z * gridDim.y + seg) * C + c] = sum;
    }
}

// Start states of the K segments of one (batch, head) and the final state.  States are [value i][key j], the
// decay acts on the key index.  grid (H, B), 256 threads, 16 elements each.
__global__ void __launch_bounds__(256) segment_states_kernel(int H, int N, int K, int slices, const float* __restrict__ s0,
                                                             const float* __restrict__ L, const float* __restrict__ Dp,
                                                             float* __restrict__ start, float* __restrict__ sT) {
    const int h = blockIdx.x, b = blockIdx.y, C = H * N, NN = N * N;
    const i64 slice_stride = (i64)gridDim.y * K * C;
    for (int e = threadIdx.x; e < NN; e += 256) {
        const int j = e % N;
        float cur = s0 ? s0[(i64)(b * H + h) * NN + e] : 0.f;
        for (int k = 0; k < K; ++k) {
            const i64 seg = (i64)b * K + k;
            start[(seg * H + h) * NN + e] = cur;
            float dl = 0.f;
            for (int z = 0; z < slices; ++z) dl += Dp[z * slice_stride + seg * C + h * N + j];
            cur = fmaf(cur, exp2f(dl), L[(seg * H + h) * NN + e]);
        }
        if (sT) sT[(i64)(b * H + h) * NN + e] = cur;
    }
}

}  // namespace

constexpr int kMaxSlices = 32;   // token slices of a segment in the decay sums

size_t wkv6_tsplit_bytes(int B, int C, int H, int K) {
    const size_t N = (size_t)(C / H);
    return ((size_t)2 * B * K * H * N * N + (size_t)kMaxSlices * B * K * C) * sizeof(float);
}

int wkv6_tsplit_states(int B, int T, int C, int H, int K, const void* w, int w_mode, const float* s0, float* work,
                       float* sT, cudaStream_t st) {
    const int N = C / H, Tseg = T / K;
    float* L = work;
    float* start = L + (size_t)B * K * H * N * N;
    float* Dl = start + (size_t)B * K * H * N * N;
    const int slices = w_mode >= 2 ? 1 : max(1, min(kMaxSlices, Tseg / 64));
    dim3 g1((C + 127) / 128, B * K, slices), b1(128, 8);
    switch (w_mode) {
        case 0: segment_decay_kernel<0><<<g1, b1, 0, st>>>(Tseg, C, w, Dl); break;
        case 1: segment_decay_kernel<1><<<g1, b1, 0, st>>>(Tseg, C, w, Dl); break;
        case 2: segment_decay_kernel<2><<<g1, b1, 0, st>>>(Tseg, C, w, Dl); break;
        default: segment_decay_kernel<3><<<g1, b1, 0, st>>>(Tseg, C, w, Dl); break;
    }
    if (int e = check_launch("wkv6_tsplit(segment decays)")) return e;
    segment_states_kernel<<<dim3(H, B), 256, 0, st>>>(H, N, K, slices, s0, L, Dl, start, sT);
    return check_launch("wkv6_tsplit(segment states)");
}

}  // namespace rwkvb200
