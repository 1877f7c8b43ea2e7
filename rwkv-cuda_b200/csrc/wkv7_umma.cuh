// tcgen05 / tensor-memory building blocks shared by the RWKV-7 kernels that run their K=64 and
// K=32 products on the 5th-generation tensor core (kind::tf32, M = 64, cta_group::1).
//
// Facts these helpers rely on (each checked on a B200 before use):
//   * an M=64 accumulator occupies lanes 0-15 of each 32-lane quarter of tensor memory: row m lives
//     at lane m%16 + 32*(m/16), column n at column n; warp w of a CTA can access quarter w only;
//   * tcgen05.ld/st with shape 16x256b moves one 16-row x 8-column tile per warp in exactly the
//     accumulator-fragment layout of mma.sync m16n8 (d0=(g,2t) d1=(g,2t+1) d2=(g+8,2t) d3=(g+8,2t+1));
//   * an accumulator can be the A operand of a later tcgen05.mma as it stands (address = its first column);
//   * shared-memory operands, K-major without swizzle: 16-byte pieces of K; piece kc of row r at
//     kc*LBO + r*16 bytes, 8-row groups SBO = 128 bytes apart; one instruction consumes K = 8 (two pieces).
// Every mbarrier wait is bounded.
#pragma once
#include "chunk_tf32.cuh"

namespace rwkvb200 {
namespace v7u {

using namespace v7c;

constexpr int LBO_T = 32 * 16 + 16;   // token-major operands [32 rows][K=64]: bytes between K pieces
constexpr int LBO_C = 64 * 16 + 16;   // channel-major operands [64 rows][K=32]

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(128 >> 4) << 32;       // SBO: 8-row groups are 128 bytes apart
    d |= (uint64_t)1 << 46;                // descriptor version of sm_100
    return d;                              // no swizzle, base offset 0
}
__device__ __forceinline__ uint32_t umma_idesc(int n) {   // D fp32, A/B tf32, both K-major, M = 64
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | (4u << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit = 1 << 20) {
    uint32_t done = 0;
    for (int it = 0; it < limit && !done; ++it)
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// one 16x256b tile (8 columns) <-> an mma.sync accumulator tile d[4]
__device__ __forceinline__ void tmem_ld8(float (&d)[4], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x1.b32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const float (&d)[4]) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x1.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "f"(d[0]), "f"(d[1]), "f"(d[2]), "f"(d[3]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// byte offset of element (row, k) in a canonical K-major array
__device__ __forceinline__ int canon(int row, int k, int lbo) { return (k >> 2) * lbo + row * 16 + (k & 3) * 4; }

}  // namespace v7u
}  // namespace rwkvb200
