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

// tensor-core path (bf16, head size 64, chunk 16, 16-byte aligned tensors)
int wkv7_chunked_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k,
                         const void* v, const void* a, const void* b, void* y, float* sT, float* s, float* sa,
                         cudaStream_t st);
// tcgen05 forward (same saved-buffer layout as the mma.sync chunked kernels) and its error word
int wkv7_umma_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k,
                      const void* v, const void* a, const void* b, void* y, float* sT, float* s, float* sa,
                      cudaStream_t st);
int wkv7_umma_error();
// the same forward as a producer/consumer pair of warp groups (one CTA per SM; for small grids)
int wkv7_umma_split_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k,
                            const void* v, const void* a, const void* b, void* y, float* sT, float* s, float* sa,
                            cudaStream_t st);
int wkv7_umma_split_error();
int wkv7_umma_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v,
                       const void* a, const void* b, const void* dy, const float* dsT, const float* s,
                       const float* sa, float* ds0, void* dr, void* dw, void* dk, void* dv, void* da, void* db,
                       cudaStream_t st);
int wkv7_umma_bwd_error();

// the same backward as a producer/consumer pair of warp groups (one CTA per SM; for small grids)
int wkv7_split_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v,
                        const void* a, const void* b, const void* dy, const float* dsT, const float* s,
                        const float* sa, float* ds0, void* dr, void* dw, void* dk, void* dv, void* da, void* db,
                        cudaStream_t st);

int wkv7_chunked_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v,
                          const void* a, const void* b, const void* dy, const float* dsT, const float* s,
                          const float* sa, float* ds0, void* dr, void* dw, void* dk, void* dv, void* da, void* db,
                          cudaStream_t st);

// 32-token chunks, every product on tcgen05 with the dependent products chained through tensor memory.
// Saved buffer: chunk-start states every 32 tokens in `s` (first half), `sa` unused.
int wkv7_l32_forward(int B, int T, int H, const float* s0, const void* r, const void* w, const void* k, const void* v,
                     const void* a, const void* b, void* y, float* sT, float* s, float* sa, cudaStream_t st);
int wkv7_l32_fwd_error();
int wkv7_l32_backward(int B, int T, int H, const void* r, const void* w, const void* k, const void* v, const void* a,
                      const void* b, const void* dy, const float* dsT, const float* s, float* ds0, void* dr, void* dw,
                      void* dk, void* dv, void* da, void* db, cudaStream_t st);
int wkv7_l32_bwd_error();

}  // namespace rwkvb200
