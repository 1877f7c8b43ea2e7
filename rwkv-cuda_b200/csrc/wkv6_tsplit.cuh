// Helpers of the time-split forward (wkv6_tsplit.cu): work-buffer layout and the segment start states.
#pragma once
#include "common.cuh"

namespace rwkvb200 {

// bytes of the work buffer: [L: B*K*H*N*N][start: B*K*H*N*N][log2 decay sums: 32 slices x B*K*C], fp32
size_t wkv6_tsplit_bytes(int B, int C, int H, int K);
// From the local end states L (front of `work`, written by the states-only pass over the (B*K, T/K, C) view):
// the decay product of every segment, the start state of every segment (second part of `work`) and the final
// state sT (optional).  w / w_mode: the decay input in the forms of the chunked kernels.
int wkv6_tsplit_states(int B, int T, int C, int H, int K, const void* w, int w_mode, const float* s0, float* work,
                       float* sT, cudaStream_t st);

}  // namespace rwkvb200
