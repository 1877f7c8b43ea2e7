// TEST INFRASTRUCTURE ONLY.  C-linkage doors onto the reference project's RWKV-5 bf16 host launchers
// (wkv5_bf16/cuda/wkv5_cuda_v1b.cu:179-191), compiled with -D_N_=64 from the reference checkout by
// oracle/build_ref.py into oracle/_ref/librwkv5_ref.so.  Nothing of the reference is copied here.
#include "ATen/ATen.h"
typedef at::BFloat16 bf16;

void cuda_forward(int B, int T, int C, int H, bf16* r, bf16* k, bf16* v, float* w, bf16* u, bf16* y);
void cuda_backward(int B, int T, int C, int H, bf16* r, bf16* k, bf16* v, float* w, float* ww, bf16* u, bf16* gy,
                   bf16* gr, bf16* gk, bf16* gv, bf16* gw, bf16* gu);

extern "C" void ref_wkv5_forward(int B, int T, int C, int H, void* r, void* k, void* v, float* w, void* u, void* y) {
    cuda_forward(B, T, C, H, (bf16*)r, (bf16*)k, (bf16*)v, w, (bf16*)u, (bf16*)y);
}
extern "C" void ref_wkv5_backward(int B, int T, int C, int H, void* r, void* k, void* v, float* w, float* ww, void* u,
                                  void* gy, void* gr, void* gk, void* gv, void* gw, void* gu) {
    cuda_backward(B, T, C, H, (bf16*)r, (bf16*)k, (bf16*)v, w, ww, (bf16*)u, (bf16*)gy, (bf16*)gr, (bf16*)gk,
                  (bf16*)gv, (bf16*)gw, (bf16*)gu);
}
