// TEST INFRASTRUCTURE ONLY.  C-linkage doors onto the reference project's own RWKV-7 host
// launchers (rwkv7_fast_fused/cuda/rwkv7_statepassing_clampw.cu:82-85,189-193), so that the
// GPU tests and the benchmark can run the unmodified reference kernel beside the library's
// kernel on the same inputs: for the "no worse than the reference kernel's error" check and
// as the on-box speed comparison.  The reference source is compiled from where it lies in the
// reference checkout (see oracle/build_ref.py); nothing of it is copied here.
#include <cuda_bf16.h>
using bf = __nv_bfloat16;

void cuda_forward(int B, int T, int H, float* s0, bf* r, bf* w, bf* k, bf* v, bf* a, bf* b, bf* y, float* sT,
                  float* s, float* sa);
void cuda_backward(int B, int T, int H, bf* r, bf* w, bf* k, bf* v, bf* a, bf* b, bf* dy, float* dsT, float* s,
                   float* sa, float* ds0, bf* dr, bf* dw, bf* dk, bf* dv, bf* da, bf* db);

extern "C" void ref_rwkv7_sp_forward(int B, int T, int H, float* s0, void* r, void* w, void* k, void* v, void* a,
                                     void* b, void* y, float* sT, float* s, float* sa) {
    cuda_forward(B, T, H, s0, (bf*)r, (bf*)w, (bf*)k, (bf*)v, (bf*)a, (bf*)b, (bf*)y, sT, s, sa);
}

extern "C" void ref_rwkv7_sp_backward(int B, int T, int H, void* r, void* w, void* k, void* v, void* a, void* b,
                                      void* dy, float* dsT, float* s, float* sa, float* ds0, void* dr, void* dw,
                                      void* dk, void* dv, void* da, void* db) {
    cuda_backward(B, T, H, (bf*)r, (bf*)w, (bf*)k, (bf*)v, (bf*)a, (bf*)b, (bf*)dy, dsT, s, sa, ds0, (bf*)dr,
                  (bf*)dw, (bf*)dk, (bf*)dv, (bf*)da, (bf*)db);
}
