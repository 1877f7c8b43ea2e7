// Launchers of the RWKV-7 kernels, shared between the entry points and the kernel files.
#pragma once
#include "common.cuh"

namespace rwkvb200 {

int wkv7_generic_forward(int dtype, int B, int T, int H, int N, int chunk, const float* s0, const void* r,
                         const void* w, const void* k, const void* v, const void* a, const void* b, void* y,
                         float* sT, float* s, float* sa, cudaStream_t st);
int wkv7_generic_backward(int dtype, int B, int T, int H, int N, int chunk, const void* r, const void* w,
                          const void* k, const void* v, const void* a, const void* b, const void* dy,
                          const float* dsT, const float* s, const float* sa, float* ds0, void* dr, void* dw, void* dk,
                          void* dv, void* da, void* db, cudaStream_t st);

// Tensor-core path (bf16, head size 64, checkpoint stride 16, 16-byte aligned tensors): chunks of 32 tokens,
// every product on tcgen05 with the dependent products chained through tensor memory.  Saved buffer: the
// state at the start of every 32-token chunk in s[b][h][c] (c < ceil(T/32); the rest of `s` and all of `sa`
// stay untouched).  `test_expire` != 0 makes the first wait of the forward run out on purpose (nothing is
// in flight: the product it waits for is not issued), to exercise the bounded-wait path.
int wkv7_l32_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k, const void* v,
                     const void* a, const void* b, void* y, float* sT, float* s, int test_expire, cudaStream_t st);
int wkv7_l32_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v, const void* a,
                      const void* b, const void* dy, const float* dsT, const float* s, float* ds0, void* dr, void* dw,
                      void* dk, void* dv, void* da, void* db, cudaStream_t st);
// The backward as two warp groups working on consecutive chunks (one thread block per SM; same
// products, results equal to rounding); for launches with at most one unit per SM.  Error word: read (clear = 0) or reset (clear = 1).
int wkv7_l32_backward_pipelined(int B, int T, int H, const void* r, const void* w, const void* k, const void* v, const void* a,
                                const void* b, const void* dy, const float* dsT, const float* s, float* ds0, void* dr, void* dw,
                                void* dk, void* dv, void* da, void* db, cudaStream_t st);
int wkv7_l32_bwdp_error(int clear);
// the forward in the same two-stage form (front: operands, U, inverses; back: the dependent chain, y, state)
int wkv7_l32_forward_pipelined(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k, const void* v,
                               const void* a, const void* b, void* y, float* sT, float* s, cudaStream_t st);
int wkv7_l32_fwdp_error(int clear);
// A tensor map over a (rows, cols) bf16 tensor with a box of [32 rows][64 columns] (one chunk of one head), made with
// cuTensorMapEncodeTiled obtained through the runtime; false when the driver has no such entry point or refuses
// the shape or the alignment.  `map` points at a CUtensorMap (128 bytes, 64-byte aligned).
bool wkv7_make_tile_map(void* map, const void* base, unsigned long long rows, unsigned long long cols);
// sticky per-device status words of the two kernels (0 = fine) and their reset
int wkv7_l32_fwd_error();
int wkv7_l32_bwd_error();
int wkv7_l32_clear_errors();

}  // namespace rwkvb200
