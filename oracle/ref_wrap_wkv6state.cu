// TEST INFRASTRUCTURE ONLY.  C-linkage doors onto the reference project's RWKV-6-with-state host launchers
// (wkv6_state/cuda/wkv6state_cuda_v1a.cu:295-309), compiled with -D_N_=64 -D_T_=256 (the reference bakes the
// sequence length in) from the reference checkout by oracle/build_ref.py into
// oracle/_ref/librwkv6state_ref.so.  Nothing of the reference is copied here.
#include "ATen/ATen.h"
typedef at::BFloat16 bf16;

void cuda_forward(int B, int T, int C, int H, bf16* r, bf16* k, bf16* v, bf16* w, bf16* u, bf16* z, bf16* y);
void cuda_backward(int B, int T, int C, int H, bf16* r, bf16* k, bf16* v, bf16* w, bf16* u, bf16* z, bf16* gy, bf16* gr,
                   bf16* gk, bf16* gv, bf16* gw, bf16* gu, bf16* gs);

extern "C" int ref_wkv6state_T(void) { return _T_; }
extern "C" void ref_wkv6state_forward(int B, int T, int C, int H, void* r, void* k, void* v, void* w, void* u, void* z,
                                      void* y) {
    cuda_forward(B, T, C, H, (bf16*)r, (bf16*)k, (bf16*)v, (bf16*)w, (bf16*)u, (bf16*)z, (bf16*)y);
}
extern "C" void ref_wkv6state_backward(int B, int T, int C, int H, void* r, void* k, void* v, void* w, void* u, void* z,
                                       void* gy, void* gr, void* gk, void* gv, void* gw, void* gu, void* gs) {
    cuda_backward(B, T, C, H, (bf16*)r, (bf16*)k, (bf16*)v, (bf16*)w, (bf16*)u, (bf16*)z, (bf16*)gy, (bf16*)gr,
                  (bf16*)gk, (bf16*)gv, (bf16*)gw, (bf16*)gu, (bf16*)gs);
}
