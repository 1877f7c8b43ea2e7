// Launchers of the chunked (tensor-core) RWKV-6 kernels: bf16, head size 64, T a multiple of 16.
#pragma once
#include "common.cuh"

namespace rwkvb200 {

// s0_kind: 0 none, 1 bf16, 2 fp32 (one N x N block per (batch, head), [value][key]).  w_mode: 0 = fp32
// log-decay (B,T,C), 1 = bf16 raw decay input (B,T,C), log-decay = -exp(w); static per channel
// (RWKV-5): 2 = fp32 decay value (C), 3 = fp32 log-decay (C).  y = NULL: only the states are rebuilt.  ck: optional
// fp32 (B,H,T/16,N,N) chunk-start states.  unsafe: device flag raised when a chunk's cumulative
// decay is too strong for the chunked form (the results are then invalid).
int wkv6_chunked_forward(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode,
                         const void* u, const void* s0, int s0_kind, void* y, float* sT, float* ck, int* unsafe,
                         cudaStream_t st, int flag_div = 1);   // flag_div: batch rows of this launch per caller's batch row (time-split views)

// Backward; ck are the chunk-start states written by wkv6_chunked_forward on the same inputs
// (fp32, (B,H,T/16,N,N)).  ds0_kind as s0_kind (0: no state gradient out).  gu is per batch: (B,C).
int wkv6_chunked_backward(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode,
                          const void* u, const void* gy, const float* dsT, const float* ck, void* gr, void* gk,
                          void* gv, void* gw, void* gu, void* ds0, int ds0_kind, cudaStream_t st,
                          float* gw32 = nullptr, float* gu32 = nullptr);   // optional unrounded (B,C) partials of gu (and of gw for a static decay)
// With a static decay (w_mode 2, 3) gw is summed over time into (B,C) instead of written per token.

// one slot of a ring of device flags for `unsafe` (clear it in the stream before the forward)
// The same forward (without saved chunk states) on tcgen05: 32-token chunks, three warp groups, inputs by TMA
// (wkv6_l32_fwd.cu).  Returns 1 when tensor maps cannot be made here: the caller then uses wkv6_chunked_forward.
int wkv6_l32_forward(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode, const void* u,
                     const void* s0, int s0_kind, void* y, float* sT, float* ck, int* unsafe, cudaStream_t st, int flag_div = 1);
// The backward on tcgen05 (wkv6_l32_bwd.cu); ck: chunk-start states every 32 tokens from wkv6_l32_forward.
int wkv6_l32_backward(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode, const void* u,
                      const void* gy, const float* dsT, const float* ck, void* gr, void* gk, void* gv, void* gw, void* gu,
                      void* ds0, int ds0_kind, cudaStream_t st, float* gw32 = nullptr, float* gu32 = nullptr);
int wkv6_l32_bwd_error(int clear);
// a tensor map over a (rows, cols) bf16 or fp32 tensor, box [32 rows][64 columns], no swizzle; false if it cannot be made
bool wkv6_make_tile_map(void* map, const void* base, unsigned long long rows, unsigned long long cols, bool fp32);
int wkv6_l32_error(int clear);   // sticky status word of that kernel: read (clear = 0) or reset (clear = 1)
// 0 = the mma.sync kernel of wkv6_chunked.cu for every forward, 1 (default) = the tcgen05 kernel where it applies
void wkv6_select_forward(int tcgen05);
void wkv6_select_backward(int tcgen05);
int wkv6_backward_with_states(int B, int T, int H, const void* r, const void* k, const void* v, const void* w, int w_mode,
                              const void* u, const void* s0, int s0_kind, const void* gy, const float* dsT, float* ck, void* gr,
                              void* gk, void* gv, void* gw, void* gu, void* ds0, int ds0_kind, int* unsafe, cudaStream_t st,
                              float* gw32 = nullptr, float* gu32 = nullptr);
int wkv6_forward_choice();

// the "decay too strong" flags of the calling stream: kChunkedFlagUnits ints, one per (batch, head) unit modulo that
constexpr int kChunkedFlagUnits = 1024;
int* wkv6_chunked_flag(cudaStream_t st);

}  // namespace rwkvb200
