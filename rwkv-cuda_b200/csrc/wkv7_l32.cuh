// Building blocks of the RWKV-7 kernels that work on chunks of 32 tokens with every contraction on
// the 5th-generation tensor core (tcgen05.mma kind::tf32, M = 64, cta_group::1) and the products
// chained through tensor memory: an accumulator is the A operand of the next product as it stands,
// so a chunk needs one round trip through registers per group of dependent products instead of one
// per product.
//
// Chunk algebra (head size 64, chunk of L = 32 tokens; S is [value i][key j]).  With d_t the decay,
// W_t = prod_{tau<=t} d_tau inside the chunk (W_{-1} = 1), We = W_{L-1} and
//   a~_t = a_t W_{t-1}   r~_t = r_t W_t   b~_s = b_s / W_s   k~_s = k_s / W_s
//   U_ab[s,t] = b~_s.a~_t (s<t)   U_ak[s,t] = k~_s.a~_t (s<t)   U_br[s,t] = b~_s.r~_t (s<=t)   U_kr[s,t] = k~_s.r~_t (s<=t)
//   T = (I - U_ab)^-1
// the forward is, with S0 the state at the start of the chunk, V = [v_t], SA = [S_{t-1} a_t], Y = [y_t] (64 x L):
//   SA = (S0 A~^T + V U_ak) T        Y = S0 R~^T + SA U_br + V U_kr        S_end = (S0 + SA B~ + V K~) diag(We)
// The divisions by W are safe because the soft clamp keeps d >= 0.545, so W >= 0.545^32 = 3.7e-9.
//
// Shared-memory operands.  Every operand array is a row-major [rows][64 or 32] fp32 (TF32) array
// in the "128-byte swizzle with 32-byte atoms" layout (descriptor layout type 1), the one layout
// in which kind::tf32 accepts an operand both K-major and MN-major (checked on a B200: with any
// other layout type an MN-major tf32 operand reads as zeros).  Element (row, col):
//   byte = (col/32)*rows*128 + row*128 + ((((col/8)&3) ^ (row&3)) * 32) + (col&7)*4
// i.e. halves of 32 columns, rows of 128 bytes, the four 32-byte pieces of a row XOR-ed with row&3.
// The XOR acts on address bits, so arrays start on 1024-byte boundaries.  The same array then serves
//   * K-major (rows = the M/N index, columns = K): start = base + row0*128 + (k0/32)*half + (k0%32)*4,
//     stride between 4-row groups (SBO) = 512;
//   * MN-major (rows = K, columns = the M/N index): start = base + k0*128, SBO = 512,
//     stride between 32-column halves (LBO) = rows*128;
// one instruction consumes K = 8.  So no operand is ever stored twice.
//
// Tensor memory: an M = 64 accumulator occupies lanes 0-15 of each 32-lane quarter (row m at lane
// m%16 + 32*(m/16)); warp w may touch quarter w%4 only; tcgen05.ld/st 16x256b moves 16 rows x 8
// columns per warp in the mma.sync accumulator layout d0=(g,2t) d1=(g,2t+1) d2=(g+8,2t) d3=(g+8,2t+1),
// g = lane/4, t = lane%4.  An fp32 accumulator read as an A operand is truncated to TF32.
// Ordering between dependent products: accumulation into the same accumulator is ordered by the hardware,
// but a product whose A operand is the accumulator of the product issued just before it is NOT (measured on
// a B200: with the tensor pipe backed up the consumer reads stale data; one unrelated instruction in between
// was enough in the test, which is no guarantee).  So between a product and a consumer of its accumulator the
// issuing warp commits to an mbarrier of its own and waits (ChainSync, about 100 cycles).
// Every mbarrier wait is bounded.
#pragma once
#include <cuda.h>
#include "wkv7_umma.cuh"
#include "wkv7_dispatch.cuh"

namespace rwkvb200 {
namespace v7x {

using namespace v7u;   // tf32r, fex2, frcp, bf16 helpers, mbarrier / tcgen05 wrappers

constexpr int LC = 32;            // tokens per chunk
constexpr int HALF64 = 64 * 128;  // bytes of one 32-column half of a 64-row array
constexpr int HALF32 = 32 * 128;  // ... of a 32-row array
constexpr int ARR64 = 2 * HALF64; // a [64][64] operand array
constexpr int ARR32 = 2 * HALF32; // a [32][64] operand array
constexpr int LAMP = 68;          // pitch (floats) of the plain [32][.] array of cumulative log2-decays
constexpr int UPITCH = 36;        // pitch (floats) of the plain fp32 32x32 matrices (rows 16-byte aligned)

// byte offset of element (row, col) of a swizzled operand array whose halves are `half` bytes apart
__device__ __forceinline__ int sw(int row, int col, int half) {
    return (col >> 5) * half + row * 128 + ((((col >> 3) & 3) ^ (row & 3)) << 5) + (col & 7) * 4;
}
// the same for a [.][32] array (one half)
__device__ __forceinline__ int sw32(int row, int col) { return row * 128 + ((((col >> 3) & 3) ^ (row & 3)) << 5) + (col & 7) * 4; }

__device__ __forceinline__ uint64_t desc_sw(uint32_t saddr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(512 >> 4) << 32;       // SBO: 4-row groups are 512 bytes apart
    d |= (uint64_t)1 << 46;                // descriptor version of sm_100
    d |= (uint64_t)1 << 61;                // layout type 1: 128-byte swizzle, 32-byte atoms
    return d;
}
// operand read K-major: rows row0.. are the M/N index, k0 (multiple of 8) the first K column
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int row0, int k0, int half) {
    return desc_sw(base + row0 * 128 + (k0 >> 5) * half + (k0 & 31) * 4, half);
}
// operand read MN-major: rows k0.. (multiple of 8) are K, columns 0.. the M/N index
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int k0, int half) { return desc_sw(base + k0 * 128, half); }

// D fp32, A/B tf32, M = 64; amn/bmn = 1 for an MN-major operand
__device__ __forceinline__ uint32_t idesc64(int n, int amn, int bmn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)amn << 15) | ((uint32_t)bmn << 16) | ((uint32_t)(n >> 3) << 17) | (4u << 24);
}

// NT consecutive 16x256b tiles (8 columns each)
template <int NT>
__device__ __forceinline__ void tmem_ld_tiles(float (*d)[4], uint32_t taddr) {
    if constexpr (NT == 4) {
        asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                     : "=f"(d[0][0]), "=f"(d[0][1]), "=f"(d[0][2]), "=f"(d[0][3]), "=f"(d[1][0]), "=f"(d[1][1]), "=f"(d[1][2]), "=f"(d[1][3]),
                       "=f"(d[2][0]), "=f"(d[2][1]), "=f"(d[2][2]), "=f"(d[2][3]), "=f"(d[3][0]), "=f"(d[3][1]), "=f"(d[3][2]), "=f"(d[3][3])
                     : "r"(taddr));
    } else if constexpr (NT == 2) {
        asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=f"(d[0][0]), "=f"(d[0][1]), "=f"(d[0][2]), "=f"(d[0][3]), "=f"(d[1][0]), "=f"(d[1][1]), "=f"(d[1][2]), "=f"(d[1][3])
                     : "r"(taddr));
    } else {
#pragma unroll
        for (int nt = 0; nt < NT; nt += 4) tmem_ld_tiles<4>(d + nt, taddr + nt * 8);
    }
}
template <int NT>
__device__ __forceinline__ void tmem_st_tiles(uint32_t taddr, const float (*d)[4]) {
    if constexpr (NT == 4) {
        asm volatile("tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                     ::"r"(taddr), "f"(d[0][0]), "f"(d[0][1]), "f"(d[0][2]), "f"(d[0][3]), "f"(d[1][0]), "f"(d[1][1]), "f"(d[1][2]), "f"(d[1][3]),
                       "f"(d[2][0]), "f"(d[2][1]), "f"(d[2][2]), "f"(d[2][3]), "f"(d[3][0]), "f"(d[3][1]), "f"(d[3][2]), "f"(d[3][3])
                     : "memory");
    } else {
#pragma unroll
        for (int nt = 0; nt < NT; nt += 4) tmem_st_tiles<4>(taddr + nt * 8, d + nt);
    }
}

// MMA issue from warp-uniform code: the whole warp runs the descriptor arithmetic (which then stays in
// uniform registers, measured 33 -> 25 cycles per instruction against a one-thread branch), the
// instruction itself is predicated on the elected lane `lead`.
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred = 0;
    asm volatile("{\n.reg .pred P1;\nelect.sync _|P1, 0xffffffff;\nselp.u32 %0, 1, 0, P1;\n}\n" : "=r"(pred));
    return pred;
}
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc, uint32_t lead) {
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n@q tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(lead) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc, uint32_t lead) {
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n@q tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc), "r"(lead) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar, uint32_t lead) {
    asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %1, 0;\n@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n"
                 ::"r"(smem_u32(bar)), "r"(lead) : "memory");
}

// The issuing warp's own barrier between a product and the consumers of its accumulator.
struct ChainSync {
    uint64_t* bar;
    uint32_t par;
    int fail;
    __device__ __forceinline__ void commit(uint32_t lead) { mma_commit(bar, lead); }
    __device__ __forceinline__ void wait() {
        if (!mbar_wait(bar, par)) fail = 1;
        par ^= 1;
        tc_fence_after();
    }
    __device__ __forceinline__ void sync(uint32_t lead) { commit(lead); wait(); }
};

__device__ __forceinline__ void mbar_init(uint64_t* bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar))); }

// barrier among `nthreads` threads: the whole CTA (id 0) or a named barrier of a warp group
__device__ __forceinline__ void group_sync(int id, int nthreads) {
    if (id == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// A [32 tokens][64 channels] bf16 tile (4 KB) for an output whose elements come out of tensor memory one
// (token, channel) at a time: written as two-byte words, read back as 16-byte pieces that go to global memory as
// whole pieces of a row.  The pieces of a row are XOR-ed with the token so that neither side has bank conflicts.
__device__ __forceinline__ int stage_off(int tt, int ch) { return tt * 128 + ((((ch >> 3) ^ tt) & 7) << 4) + (ch & 7) * 2; }
// thread idx (0..255) = (token, piece): the piece of the staged tile -> out[(token0 + token) * C + 8 * piece ..]
__device__ __forceinline__ void stage_flush(const unsigned char* stage, bf16* out, i64 row0_off, int C, int idx, int valid) {
    const int tt = idx >> 3, piece = idx & 7;
    if (tt < valid)
        *reinterpret_cast<uint4*>(out + row0_off + (i64)tt * C + piece * 8) =
            *reinterpret_cast<const uint4*>(stage + tt * 128 + ((piece ^ (tt & 7)) << 4));
}

// ---- the part of a chunk that does not depend on the carried state ---------------------------------
// Raw inputs of one chunk as loaded by a thread: channels (2*lane, 2*lane+1) of TPW consecutive tokens
// (token index inside the chunk = TPW*warp + q).  NX tensors: r w k v a b [dy].
template <int NX, int TPW>
struct RawChunk {
    uint32_t x[NX][TPW];
};

// Loads the thread's part of chunk c; tokens at or beyond T read as zeros (a zero raw decay input is
// replaced by "no decay" in prepare_operands through the `valid` count).
template <int NX, int TPW>
__device__ __forceinline__ void fetch_chunk(RawChunk<NX, TPW>& rc, const bf16* const* src, i64 tok0, int C, int c, int T,
                                            int warp, int lane) {
    const int t0 = c * LC + TPW * warp;
    const i64 off = tok0 + (i64)t0 * C + 2 * lane;
#pragma unroll
    for (int x = 0; x < NX; ++x)
#pragma unroll
        for (int q = 0; q < TPW; ++q)
            rc.x[x][q] = (t0 + q < T) ? __ldg(reinterpret_cast<const unsigned int*>(src[x] + off + (i64)q * C)) : 0u;
}

// Asks for the inputs of a chunk to be brought into L2 ahead of the loads above: one [32 tokens][64 channels] tile per
// tensor through its tensor map (x = first channel, y = first row of the (B*T, C) view) and `state_bytes` at `state`
// (16-byte aligned).  Called by one thread, two chunks ahead of the chunk being worked on.  Measured on a B200 with two
// thread blocks per SM: backward of B16 T4096 4.43 -> 4.34 ms.  (One request per row, 128 bytes each, costs more
// than it saves: about 60 cycles of the copy engine per request.  With one thread block per SM nothing is gained.)
template <int NX>
struct TileMaps {
    CUtensorMap m[NX];
    int valid;   // 0: no maps could be made, nothing is requested
};
// One [32 rows][64 columns] tile of a tensor map (x = first column, y = first row) -> shared memory as plain rows, by
// the copy engine; completion is counted in bytes on the mbarrier, on which one thread has announced them before.
__device__ __forceinline__ void tma_tile_load(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void mbar_expect_bytes(uint64_t* bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void l2_prefetch_tile(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "r"(bytes) : "memory");
}
// host side: maps over NX (B*T, C) bf16 tensors; valid = 0 when any of them cannot be made
template <int NX>
inline void make_tile_maps(TileMaps<NX>& maps, const void* const* tensors, int B, int T, int H) {
    maps.valid = 1;
    for (int x = 0; x < NX && maps.valid; ++x)
        if (!wkv7_make_tile_map(&maps.m[x], tensors[x], (unsigned long long)B * T, (unsigned long long)H * 64)) maps.valid = 0;
}
template <int NX>
__device__ __forceinline__ void prefetch_chunk_l2(const TileMaps<NX>& maps, int x, int y, const void* state, uint32_t state_bytes) {
    if (!maps.valid) return;
#pragma unroll
    for (int q = 0; q < NX; ++q) l2_prefetch_tile(&maps.m[q], x, y);
    if (state != nullptr && (reinterpret_cast<uintptr_t>(state) & 15) == 0) l2_prefetch(state, state_bytes);
}

// Writes the scaled operands of the chunk:
//   AR rows 0-31 = a~_t, rows 32-63 = r~_t        BK rows 0-31 = b~_t, rows 32-63 = k~_t      (columns = key channel)
//   V rows = v_t (dst_v, a 32-row half-array pair at the given half stride), optionally dY the same way,
//   We[j] = decay over the whole chunk, and optionally the cumulative log2-decays lam[t][j] (plain [32][LAMP]).
// Tokens at or beyond `valid` (counted inside the chunk) are neutral: no decay, zero vectors.
// Hs is a [NW][64] exchange buffer.  Contains one barrier among the NW calling warps (the CTA, or the named
// barrier `bar_id` of a warp group); the caller synchronises afterwards.
template <int NX, int TPW, int NW>
__device__ __forceinline__ void prepare_operands(const RawChunk<NX, TPW>& rc, int valid, unsigned char* AR, unsigned char* BK,
                                                 unsigned char* dstV, int halfV, unsigned char* dstDY, int halfDY,
                                                 float* We, float* Hs, float* lam_out, int warp, int lane, int bar_id = 0) {
    const int j0 = 2 * lane, t0 = TPW * warp;
    float cs[TPW][2];
    float run0 = 0.f, run1 = 0.f;
#pragma unroll
    for (int q = 0; q < TPW; ++q) {
        const float2 x = bf16x2_to_f2(rc.x[1][q]);
        if (t0 + q < valid) {
            run0 = fmaf(kWScale2, frcp(1.f + fexp(-x.x)), run0);
            run1 = fmaf(kWScale2, frcp(1.f + fexp(-x.y)), run1);
        }
        cs[q][0] = run0; cs[q][1] = run1;
    }
    *reinterpret_cast<float2*>(Hs + warp * 64 + j0) = make_float2(run0, run1);
    group_sync(bar_id, NW * 32);
    float base0 = 0.f, base1 = 0.f, tot0 = 0.f, tot1 = 0.f;
#pragma unroll
    for (int gq = 0; gq < NW; ++gq) {
        const float2 h = *reinterpret_cast<const float2*>(Hs + gq * 64 + j0);
        if (gq < warp) { base0 += h.x; base1 += h.y; }
        tot0 += h.x; tot1 += h.y;
    }
    if (warp == 0) *reinterpret_cast<float2*>(We + j0) = make_float2(fex2(tot0), fex2(tot1));
    float wp0 = fex2(base0), wp1 = fex2(base1);
#pragma unroll
    for (int q = 0; q < TPW; ++q) {
        const int tt = t0 + q;
        const float lam0 = base0 + cs[q][0], lam1 = base1 + cs[q][1];
        const float wt0 = fex2(lam0), wt1 = fex2(lam1), iw0 = fex2(-lam0), iw1 = fex2(-lam1);
        const float2 r2 = bf16x2_to_f2(rc.x[0][q]), k2 = bf16x2_to_f2(rc.x[2][q]), v2 = bf16x2_to_f2(rc.x[3][q]);
        const float2 a2 = bf16x2_to_f2(rc.x[4][q]), b2 = bf16x2_to_f2(rc.x[5][q]);
        *reinterpret_cast<float2*>(AR + sw(tt, j0, HALF64)) = make_float2(tf32rf(a2.x * wp0), tf32rf(a2.y * wp1));
        *reinterpret_cast<float2*>(AR + sw(32 + tt, j0, HALF64)) = make_float2(tf32rf(r2.x * wt0), tf32rf(r2.y * wt1));
        *reinterpret_cast<float2*>(BK + sw(tt, j0, HALF64)) = make_float2(tf32rf(b2.x * iw0), tf32rf(b2.y * iw1));
        *reinterpret_cast<float2*>(BK + sw(32 + tt, j0, HALF64)) = make_float2(tf32rf(k2.x * iw0), tf32rf(k2.y * iw1));
        *reinterpret_cast<float2*>(dstV + sw(tt, j0, halfV)) = v2;
        if constexpr (NX > 6) {
            *reinterpret_cast<float2*>(dstDY + sw(tt, j0, halfDY)) = bf16x2_to_f2(rc.x[6][q]);
        }
        if (lam_out != nullptr) *reinterpret_cast<float2*>(lam_out + tt * LAMP + j0) = make_float2(lam0, lam1);
        wp0 = wt0; wp1 = wt1;
    }
}

// U = [B~;K~] [A~;R~]^T on the tensor core: D rows 0-31 = b~_s, 32-63 = k~_s; columns 0-31 = a~_t, 32-63 = r~_t.
__device__ __forceinline__ void issue_u(uint32_t d_tmem, uint32_t ar, uint32_t bk, uint32_t lead) {
    const uint32_t id = idesc64(64, 0, 0);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) mma_ss(d_tmem, desc_k(bk, 0, ks * 8, HALF64), desc_k(ar, 0, ks * 8, HALF64), id, ks > 0, lead);
}

// One warp's 16 rows of U (all 64 columns, tiles u[0..7]) -> masked matrices.  quarter 0,1: rows b~_s
// (s = 16*quarter + g / + 8): U_ab (strict; plain fp32 [32][UPITCH] for the inverses of its diagonal
// blocks, and its upper right 16x16 block into the swizzled TF32 [32][32] operand N1, whose other blocks
// stay zero) and U_br (s <= t);
// quarter 2,3: rows k~_s: U_ak (strict) and U_kr (s <= t).  U_ak, U_br, U_kr go to swizzled [32][32]
// operand arrays, TF32.
__device__ __forceinline__ void scatter_u(const float (*u)[4], int quarter, int lane, float* Uab, unsigned char* N1,
                                          unsigned char* Uak, unsigned char* Ubr, unsigned char* Ukr) {
    const int g = lane >> 2, t = lane & 3;
    const int sb = 16 * (quarter & 1) + g;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int s = sb + 8 * h, c0 = nt * 8 + 2 * t;
            const float a0 = s < c0 ? u[nt][2 * h] : 0.f, a1 = s < c0 + 1 ? u[nt][2 * h + 1] : 0.f;           // vs a~: strict
            const float r0 = s <= c0 ? u[4 + nt][2 * h] : 0.f, r1 = s <= c0 + 1 ? u[4 + nt][2 * h + 1] : 0.f;  // vs r~
            if (quarter < 2) {
                *reinterpret_cast<float2*>(Uab + s * UPITCH + c0) = make_float2(a0, a1);
                if (quarter == 0 && nt >= 2) *reinterpret_cast<float2*>(N1 + sw32(s, c0)) = make_float2(tf32rf(a0), tf32rf(a1));
                *reinterpret_cast<float2*>(Ubr + sw32(s, c0)) = make_float2(tf32rf(r0), tf32rf(r1));
            } else {
                *reinterpret_cast<float2*>(Uak + sw32(s, c0)) = make_float2(tf32rf(a0), tf32rf(a1));
                *reinterpret_cast<float2*>(Ukr + sw32(s, c0)) = make_float2(tf32rf(r0), tf32rf(r1));
            }
        }
}

// Inverse of a 16x16 unit upper triangular block: T = (I - U)^-1 for the strictly upper triangular 16x16
// block that starts at Ub (plain fp32, pitch PITCH floats, rows 16-byte aligned); result rounded to TF32
// into the diagonal block at (r0, r0) of the swizzled [32][32] operand array D0 (whose off-diagonal blocks
// stay zero).  Back substitution in fp32, lane t (< 16) owns column t:
//   T[s,t] = [s == t] + sum_{m>s} U[s,m] T[m,t]      (rows s = 14 .. 0; zero below the diagonal by itself)
// Software-pipelined: the sum of row s is split into its newest term (m = s+1), the second newest (m = s+2)
// and the rest (m >= s+3); the rest of row s-1 is accumulated between the two final FMAs of row s, so one
// FMA per row sits on the dependent chain, and rows are fetched (float4) three rows ahead.  Measured alone
// on a B200: 530 cycles against 620 for the plain loop.  Called by one full warp.
template <int PITCH>
__device__ __forceinline__ void tri_inverse16(const float* Ub, unsigned char* Tsw, int r0, int lane) {
    constexpr int Lb = 16;
    const int t = lane & 15;
    float col[Lb], tp[Lb];
    float4 rw[Lb][4];
#pragma unroll
    for (int s = 0; s < Lb; ++s) tp[s] = (s == t) ? 1.f : 0.f;
    col[Lb - 1] = tp[Lb - 1];
    auto load_row = [&](int s) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (4 * q + 3 >= s + 1) rw[s][q] = *reinterpret_cast<const float4*>(Ub + s * PITCH + 4 * q);
    };
    auto u = [&](int s, int m) {
        const float4 rr = rw[s][m >> 2];
        return (m & 3) == 0 ? rr.x : (m & 3) == 1 ? rr.y : (m & 3) == 2 ? rr.z : rr.w;
    };
    load_row(14); load_row(13); load_row(12);
#pragma unroll
    for (int s = Lb - 2; s >= 0; --s) {
        if (s >= 3) load_row(s - 3);
        float x = tp[s];
        if (s + 2 < Lb) x = fmaf(u(s, s + 2), col[s + 2], x);
        if (s >= 1) {
            float a0 = tp[s - 1], a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int m = s + 2; m < Lb; ++m) {
                const float uu = u(s - 1, m);
                if ((m & 3) == 0) a0 = fmaf(uu, col[m], a0);
                else if ((m & 3) == 1) a1 = fmaf(uu, col[m], a1);
                else if ((m & 3) == 2) a2 = fmaf(uu, col[m], a2);
                else a3 = fmaf(uu, col[m], a3);
            }
            tp[s - 1] = (a0 + a1) + (a2 + a3);
        }
        col[s] = fmaf(u(s, s + 1), col[s + 1], x);
    }
    if (lane < 16) {
#pragma unroll
        for (int s = 0; s < Lb; ++s) *reinterpret_cast<float*>(Tsw + sw32(r0 + s, r0 + t)) = tf32rf(col[s]);
    }
}

// SA = Z (I - U_ab)^-1 on the tensor core, all in tensor memory.  With blocks of 16 tokens,
//   (I - U_ab)^-1 = D0 + D0 N1 D0,   D0 = diag(T00, T11) (inverses of the diagonal blocks),  N1 = [[0, U01], [0, 0]]
// so  Q = Z D0,  R = Q N1 (only rows 0-15 of N1 are non-zero),  SA = Q + R D0 (only columns 16-31 of R are non-zero).
// Every product has N = 32 and starts at the first column of its accumulator.  tmZ: 32 columns holding Z
// (complete when called; overwritten by R), tmSA: 32 columns receiving SA (complete on return); d0/n1:
// swizzled [32][32] operands read MN-major.  `between()` is issued after the first product's commit and
// before the wait on it (independent work that hides the wait).
template <class F>
__device__ __forceinline__ void issue_solve(uint32_t tmSA, uint32_t tmZ, uint32_t d0, uint32_t n1, uint32_t lead, ChainSync& cs, F between) {
    const uint32_t id = idesc64(32, 0, 1);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) mma_ts(tmSA, tmZ + ks * 8, desc_mn(d0, ks * 8, HALF32), id, ks > 0, lead);
    cs.commit(lead);
    between();
    cs.wait();
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) mma_ts(tmZ, tmSA + ks * 8, desc_mn(n1, ks * 8, HALF32), id, ks > 0, lead);
    cs.sync(lead);
#pragma unroll
    for (int ks = 2; ks < 4; ++ks) mma_ts(tmSA, tmZ + ks * 8, desc_mn(d0, ks * 8, HALF32), id, 1, lead);
    cs.sync(lead);
}
// The same for the transposed system, EV = EV0 (I - U_ab)^-T = Q + (Q N1^T) D0^T with Q = EV0 D0^T
// (only rows 16-31 of N1^T and columns 0-15 of the middle product are non-zero); operands read K-major.
template <class F>
__device__ __forceinline__ void issue_solve_t(uint32_t tmEV, uint32_t tmEV0, uint32_t d0, uint32_t n1, uint32_t lead, ChainSync& cs, F between) {
    const uint32_t id = idesc64(32, 0, 0);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) mma_ts(tmEV, tmEV0 + ks * 8, desc_k(d0, 0, ks * 8, HALF32), id, ks > 0, lead);
    cs.commit(lead);
    between();
    cs.wait();
#pragma unroll
    for (int ks = 2; ks < 4; ++ks) mma_ts(tmEV0, tmEV + ks * 8, desc_k(n1, 0, ks * 8, HALF32), id, ks > 2, lead);
    cs.sync(lead);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) mma_ts(tmEV, tmEV0 + ks * 8, desc_k(d0, 0, ks * 8, HALF32), id, 1, lead);
    cs.sync(lead);
}

}  // namespace v7x
}  // namespace rwkvb200
