/*
 * rwkvb200 — C ABI of the B200 (sm_100a) WKV / depthwise_conv1d kernels.
 *
 * Every entry point replaces one `cuda_forward` / `cuda_backward` host launcher of
 * BlinkDL/RWKV-CUDA (cited per function, paths inside that project) and is what that
 * project's pybind / TORCH_LIBRARY bindings would call instead.
 *
 * Conventions
 *   - plain device pointers and sizes only; all tensors contiguous row-major;
 *   - all buffers are caller-owned and the library allocates nothing.  What it keeps between calls:
 *     the RWKV-7 kernel choice (rwkvb200_wkv7_select_path, process-wide, atomic), a sticky
 *     per-device status word written by the tcgen05 kernels when a bounded wait runs out
 *     (rwkvb200_device_status / _clear), per-stream flag slots of the chunked RWKV-5/6 kernels and
 *     the fixed scratch array of rwkvb200_wkv6_backward_noalloc;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *     kernels are enqueued, not waited for;
 *   - return value: RWKVB200_OK or a negative RWKVB200_E* code; nothing aborts, nothing
 *     traps on the device.  rwkvb200_strerror() gives a message for a code and
 *     rwkvb200_last_error() the detail text of the calling thread's last failure.
 *   - `dtype` selects the element type of the activation tensors (RWKVB200_F32 or
 *     RWKVB200_BF16); recurrent state and all accumulation are fp32.
 *   - head size N = C / H may be any value in 1..128 (the reference bakes it in with -D_N_).
 */
#ifndef RWKVB200_H
#define RWKVB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RWKVB200_OK 0
#define RWKVB200_EINVAL (-1)      /* bad size / combination of arguments            */
#define RWKVB200_ENULL (-2)       /* required pointer is NULL                       */
#define RWKVB200_EALIGN (-3)      /* pointer not aligned as the kernel needs        */
#define RWKVB200_EUNSUPPORTED (-4)/* valid request, no kernel instance for it        */
#define RWKVB200_ECUDA (-5)       /* CUDA runtime reported an error at launch        */

#define RWKVB200_F32 0
#define RWKVB200_BF16 1

#define RWKVB200_MAX_HEAD_SIZE 128

const char* rwkvb200_strerror(int code);
const char* rwkvb200_last_error(void);
/* Library version, and the compute capability the kernels were built for (100). */
int rwkvb200_version(void);
int rwkvb200_built_for_sm(void);

/* ---------------------------------------------------------------------------------
 * RWKV-4 WKV, fp32.  Replaces cuda_forward / cuda_backward of wkv/cuda/wkv_cuda_v2.cu:116-130
 * (bound in wkv/cuda/wkv_op.cpp:6-11).
 *   w (C) = -exp(time_decay), u (C); k, v, y, gy, gk, gv (B,T,C).
 *   gw, gu (B,C): per-batch partial sums, ACCUMULATED into (caller zero-fills, then sums
 *   over B), gw already multiplied by w as the reference does (wkv_cuda_v2.cu:111-113).
 *   No limit on T or C (the reference requires T <= 4096).
 */
int rwkvb200_wkv4_forward(int B, int T, int C, const float* w, const float* u, const float* k,
                          const float* v, float* y, void* stream);
int rwkvb200_wkv4_backward(int B, int T, int C, const float* w, const float* u, const float* k,
                           const float* v, const float* gy, float* gw, float* gu, float* gk,
                           float* gv, void* stream);

/* ---------------------------------------------------------------------------------
 * depthwise_conv1d ("TimeX"), fp32.  Replaces cuda_forward / cuda_backward of
 * depthwise_conv1d/cuda/timex_cuda_v3.cu:140-150 (bound in timex_op.cpp:6-11).
 *   w (C,T); k, x, gwk, gk (B,C,T); gw (B,C,T) per-batch partials (caller sums over B).
 *   x[b,c,t] = eps + sum_{u<=t} w[c,(T-1)-(t-u)] k[b,c,u].
 *   Any B and T (the reference requires T%4==0, T<=Tmax, B%BF==0).
 * rwkvb200_timex_backward_reduced writes gw already summed over the batch, shape (C,T); the sum is taken in a
 * fixed order (the per-row gradients pass through the gk buffer before gk is written).
 */
int rwkvb200_timex_forward(const float* w, const float* k, float* x, float eps, int B, int C,
                           int T, void* stream);
int rwkvb200_timex_backward(const float* w, const float* k, const float* gwk, float* gw,
                            float* gk, int B, int C, int T, void* stream);
int rwkvb200_timex_backward_reduced(const float* w, const float* k, const float* gwk,
                                    float* gw_sum, float* gk, int B, int C, int T, void* stream);

/* ---------------------------------------------------------------------------------
 * RWKV-5 WKV, fp32 or bf16 activations.  Replaces cuda_forward / cuda_backward of
 * wkv5_bf16/cuda/wkv5_cuda_v1b.cu:179-191 (bf16; wkv5_op.cpp:8-13) and of
 * wkv5/cuda/wkv5_cuda_v1e.cu (fp32; wkv5/cuda/wkv5_op.cpp:6-11).
 *   r,k,v,y,gy,gr,gk,gv (B,T,C) and u (H,N) in `dtype`; w = exp(-exp(w_raw)) and
 *   ww = -exp(w_raw) as fp32 (H,N); gw, gu (B,C) per-batch partials in `dtype`
 *   (gw already multiplied by ww).
 */
int rwkvb200_wkv5_forward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                          const void* v, const float* w, const void* u, void* y, void* stream);
int rwkvb200_wkv5_backward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                           const void* v, const float* w, const float* ww, const void* u,
                           const void* gy, void* gr, void* gk, void* gv, void* gw, void* gu,
                           void* stream);
/* Sum of the per-batch parameter-gradient partials the backward kernels emit, gw / gu (B,n) in `dtype`,
 * into fp32 out[n], accumulated in fp32 in batch order (deterministic).  Replaces the harnesses'
 * `torch.sum(gw, 0)` on bf16 partials (wkv5_bf16/run.py:86-87, wkv6/run.py:169, wkv/run.py:115-116), whose
 * result is rounded to bf16; several partials can be reduced into one fp32 buffer, which is then what a
 * multi-GPU run all-reduces once. */
int rwkvb200_reduce_batch_partials(int dtype, int B, int n, const void* partial, float* out, void* stream);
/* The same backward with a caller-provided work buffer of rwkvb200_wkv5_scratch_bytes(B,T,C) bytes
 * (16 per element; contents undefined afterwards).  No counterpart in the reference.  With it,
 * bf16 / head size 64 / T a multiple of 16 runs on the chunked tensor-core kernels (RWKV-5 is
 * RWKV-6 with a decay that is constant over time; they need the chunk-start states of a forward
 * pass, which go into the buffer); other shapes, and decays too strong for the chunked form, run
 * the same kernel as rwkvb200_wkv5_backward.  The forward takes the chunked path on its own. */
size_t rwkvb200_wkv5_scratch_bytes(int B, int T, int C);
int rwkvb200_wkv5_backward_ws(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                              const void* v, const float* w, const float* ww, const void* u,
                              const void* gy, void* gr, void* gk, void* gv, void* gw, void* gu,
                              void* scratch, void* stream);
/* The same with, in addition, the (B,C) partials of gw and gu unrounded in fp32: summed over the batch with
 * rwkvb200_reduce_batch_partials they are the parameter gradients without the bf16 round trip of the reference
 * harness (wkv5_bf16/run.py:83-87). */
int rwkvb200_wkv5_backward_ws32(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                const void* v, const float* w, const float* ww, const void* u,
                                const void* gy, void* gr, void* gk, void* gv, void* gw, void* gu,
                                float* gw32, float* gu32, void* scratch, void* stream);

/* ---------------------------------------------------------------------------------
 * RWKV-5a WKV (decay w1[j]*w2[i], bonus u1[j]+u2[i]), fp32 or bf16 activations.
 * Replaces cuda_forward / cuda_backward of wkv5a/cuda/wkv5a_cuda_v1a.cu:214-226
 * (wkv5a_op.cpp:9-17; the reference instantiates DTYPE=float only).
 */
int rwkvb200_wkv5a_forward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                           const void* v, const float* w1, const void* u1, const float* w2,
                           const void* u2, void* y, void* stream);
int rwkvb200_wkv5a_backward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                            const void* v, const float* w1, const float* ww1, const void* u1,
                            const float* w2, const float* ww2, const void* u2, const void* gy,
                            void* gr, void* gk, void* gv, void* gw1, void* gu1, void* gw2,
                            void* gu2, void* stream);

/* ---------------------------------------------------------------------------------
 * RWKV-6 WKV (per-token decay), bf16 or fp32 activations.  Replaces cuda_forward /
 * cuda_backward of wkv6/cuda/wkv6_cuda_v1.cu:211-223 (wkv6_op.cpp:8-13).
 *   w (B,T,C) fp32 = -exp(w_raw) (the kernel applies exp); gw (B,T,C) in `dtype` w.r.t.
 *   w_raw; gu (B,C) per-batch partials.
 *   `scratch`: device buffer of rwkvb200_wkv6_scratch_bytes(B,T,C) bytes (16 per element) used
 *   inside the backward (contents undefined afterwards).  No limit on T (the reference's backward
 *   fails for T >= 128, wkv6/run.py:51).
 *   bf16 with head size 64 and T a multiple of 16 runs on chunked tensor-core kernels; if these
 *   meet a chunk whose cumulative decay is too strong for that form (sum of |log w| over 16 tokens
 *   above 80 in some channel) the general-shape kernels redo the call in the same stream.
 */
size_t rwkvb200_wkv6_scratch_bytes(int B, int T, int C);
int rwkvb200_wkv6_forward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                          const void* v, const float* w, const void* u, void* y, void* stream);
int rwkvb200_wkv6_backward(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                           const void* v, const float* w, const void* u, const void* gy,
                           void* gr, void* gk, void* gv, void* gw, void* gu, void* scratch,
                           void* stream);

/* RWKV-6 backward for callers that cannot allocate device memory (no counterpart in the
 * reference).  Same operator and arguments as rwkvb200_wkv6_backward minus `scratch`: the
 * intermediate buffer is a fixed 32 MiB array inside the library image, so B*T*C must not
 * exceed rwkvb200_wkv6_backward_noalloc_max_elems() (8 Mi elements); larger problems are
 * refused with RWKVB200_EINVAL.  The call allocates and frees nothing.
 *   - The first call on each device looks the array's device address up (with that device
 *     current); make that first call outside of any stream capture.
 *   - All calls share the one array and it keeps whatever the last call left in it; the kernel
 *     overwrites what it uses, so nothing needs clearing, but two calls whose kernels overlap
 *     on the GPU (different streams) race on it: serialise them.
 */
size_t rwkvb200_wkv6_backward_noalloc_max_elems(void);
int rwkvb200_wkv6_backward_noalloc(int dtype, int B, int T, int C, int H, const void* r,
                                   const void* k, const void* v, const float* w, const void* u,
                                   const void* gy, void* gr, void* gk, void* gv, void* gw, void* gu,
                                   void* stream);

/* ---------------------------------------------------------------------------------
 * RWKV-6 WKV with initial state.  Replaces cuda_forward / cuda_backward of
 * wkv6_state/cuda/wkv6state_cuda_v1a.cu:295-308 (wkv6state_op.cpp:8-13).
 *   every tensor in `dtype` including the raw decay w (B,T,C) and the state
 *   s, gs (B,H,N,N) indexed [value i][key j]; decay = exp(-exp(w)) inside the kernel.
 * The *_ex forms take the state in fp32, also return the final state sT, and accept its
 * gradient dsT (sT / dsT may be NULL): the superset needed for state passing.
 */
int rwkvb200_wkv6state_forward(int dtype, int B, int T, int C, int H, const void* r,
                               const void* k, const void* v, const void* w, const void* u,
                               const void* s, void* y, void* stream);
int rwkvb200_wkv6state_backward(int dtype, int B, int T, int C, int H, const void* r,
                                const void* k, const void* v, const void* w, const void* u,
                                const void* s, const void* gy, void* gr, void* gk, void* gv,
                                void* gw, void* gu, void* gs, void* scratch, void* stream);
int rwkvb200_wkv6state_forward_ex(int dtype, int B, int T, int C, int H, const void* r,
                                  const void* k, const void* v, const void* w, const void* u,
                                  const float* s0, void* y, float* sT, void* stream);
int rwkvb200_wkv6state_backward_ex(int dtype, int B, int T, int C, int H, const void* r,
                                   const void* k, const void* v, const void* w, const void* u,
                                   const float* s0, const void* gy, const float* dsT, void* gr,
                                   void* gk, void* gv, void* gw, void* gu, float* ds0,
                                   void* scratch, void* stream);

/* RWKV-5 training flow with saved states, as rwkvb200_wkv6state_forward_saved below: `saved` has
 * rwkvb200_wkv5_scratch_bytes(B,T,C) bytes; gw32 / gu32 (optional, both or none): the unrounded fp32 (B,C) partials. */
int rwkvb200_wkv5_forward_saved(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                const void* v, const float* w, const void* u, void* y, void* saved, void* stream);
int rwkvb200_wkv5_backward_saved(int dtype, int B, int T, int C, int H, const void* r, const void* k,
                                 const void* v, const float* w, const float* ww, const void* u,
                                 const void* gy, void* gr, void* gk, void* gv, void* gw, void* gu,
                                 float* gw32, float* gu32, void* saved, int saved_valid, void* stream);

/* RWKV-6 with fp32 state, training flow with saved states: the forward leaves the states at the start of every
 * 32-token chunk in `saved` (rwkvb200_wkv6_scratch_bytes(B,T,C) bytes of device memory, kept by the caller until the
 * backward), so that the backward need not run over the sequence once more to rebuild them.  The forward returns
 * RWKVB200_OK when it saved them, 1 when it ran on kernels that do not (pass saved_valid = 0 then: the backward behaves
 * as rwkvb200_wkv6state_backward_ex with `saved` as scratch), a negative code on error.  No counterpart in the
 * reference, whose operator recomputes everything in the backward (wkv6state_cuda_v1a.cu). */
int rwkvb200_wkv6state_forward_saved(int dtype, int B, int T, int C, int H, const void* r,
                                     const void* k, const void* v, const void* w, const void* u,
                                     const float* s0, void* y, float* sT, void* saved, void* stream);
int rwkvb200_wkv6state_backward_saved(int dtype, int B, int T, int C, int H, const void* r,
                                      const void* k, const void* v, const void* w, const void* u,
                                      const float* s0, const void* gy, const float* dsT, void* gr,
                                      void* gk, void* gv, void* gw, void* gu, float* ds0,
                                      void* saved, int saved_valid, void* stream);

/* Kernels of the bf16 / head-size-64 forward and backward of RWKV-5 and RWKV-6: 1 (default) = tcgen05 (32-token
 * chunks; the forward as three warp groups with inputs by TMA), 0 = mma.sync (16-token chunks).  Results agree to rounding.
 * Process-wide, for tests and measurements; no counterpart in the reference. */
int rwkvb200_wkv6_select_forward(int kernel);

/* Forward split over time (two-level scan): T is cut into `segments` pieces that run at the same time, for
 * launches with few (batch, head) units.  Replaces the idea of the reference's forward-only
 * wkv5_bf16/cuda/wkv5_cuda_v3.cu:12-128 (kernel_forward_accumulate_state + kernel_forward<true>), extended to
 * RWKV-6's per-token decay and to a state in / out.  bf16, head size 64, T/segments a multiple of 16,
 * 16-byte aligned tensors; `work`: rwkvb200_wkv6_tsplit_bytes(...) bytes of device memory.  Arguments otherwise
 * as rwkvb200_wkv5_forward / rwkvb200_wkv6state_forward_ex; results equal theirs to rounding. */
size_t rwkvb200_wkv6_tsplit_bytes(int B, int T, int C, int H, int segments);
int rwkvb200_wkv5_forward_tsplit(int dtype, int B, int T, int C, int H, int segments, const void* r,
                                 const void* k, const void* v, const float* w, const void* u, void* y,
                                 void* work, void* stream);
int rwkvb200_wkv6state_forward_tsplit(int dtype, int B, int T, int C, int H, int segments, const void* r,
                                      const void* k, const void* v, const void* w, const void* u,
                                      const float* s0, void* y, float* sT, void* work, void* stream);

/* ---------------------------------------------------------------------------------
 * RWKV-7 generalised delta rule with soft-clamped decay, bf16 or fp32 activations.
 * One pair of entry points serves the three reference operators:
 *   rwkv7_clampw              cuda_forward/backward, rwkv7_fast_fused/cuda/rwkv7_clampw.cu:76-79,172-176
 *                             (rwkv7_clampw.cpp:12-24):        s0 = sT = dsT = ds0 = NULL
 *   rwkv7_state_clampw        rwkv7_state_clampw.cu (rwkv7_state_clampw.cpp:12-24):  sT = dsT = NULL
 *   rwkv7_statepassing_clampw rwkv7_statepassing_clampw.cu:82-85,189-193
 *                             (rwkv7_statepassing_clampw.cpp:12-24): all four given
 *   r,w,k,v,a,b,y,dy,dr..db (B,T,H,N) in `dtype` (w is the raw decay input; the kernel
 *   computes exp(-e^{-0.5} sigmoid(w))); s0,sT,dsT,ds0 (B,H,N,N) fp32 indexed
 *   [value i][key j].
 *   s  (B,H,T/chunk_len,N,N) fp32 and sa (B,T,H,N) fp32 are the saved-for-backward buffers
 *   the reference harness allocates; forward fills them, backward reads them, their internal
 *   layout is private to this library.  T must be a multiple of chunk_len (reference: 16).
 */
int rwkvb200_wkv7_forward(int dtype, int B, int T, int H, int N, int chunk_len, const float* s0,
                          const void* r, const void* w, const void* k, const void* v,
                          const void* a, const void* b, void* y, float* sT, float* s, float* sa,
                          void* stream);
int rwkvb200_wkv7_backward(int dtype, int B, int T, int H, int N, int chunk_len, const void* r,
                           const void* w, const void* k, const void* v, const void* a,
                           const void* b, const void* dy, const float* dsT, const float* s,
                           const float* sa, float* ds0, void* dr, void* dw, void* dk, void* dv,
                           void* da, void* db, void* stream);

/* Inference-shaped RWKV-7 entry point: advances `state` (B,H,N,N) fp32, indexed [value i][key j] as the
 * reference's s0 / sT (rwkv7_fast_fused/cuda/rwkv7_statepassing_clampw.cu:26-32, 78-80), by T >= 1 tokens
 * IN PLACE and writes y (B,T,H,N).  Nothing is saved for a backward pass and T needs no alignment: T = 1
 * is one decoding step, a long T a prompt.  The reference has no such launcher (its forward always saves
 * s / sa and wants T % 16 == 0); same arithmetic as rwkvb200_wkv7_forward with s0 = sT = state. */
int rwkvb200_wkv7_state_update(int dtype, int B, int T, int H, int N, float* state, const void* r,
                               const void* w, const void* k, const void* v, const void* a, const void* b,
                               void* y, void* stream);

/* Kernel choice for RWKV-7 (process-wide; set it before launching work, not concurrently with it):
 * 0 = automatic (tensor-core kernels for bf16, N=64, chunk_len=16; general-shape kernels otherwise),
 * 1 = general-shape kernels only, 2 = tensor-core kernels or RWKVB200_EUNSUPPORTED.
 * The forward and the backward of one operator call must run under the same setting: the content
 * of s / sa differs between the two kernel families (tensor-core kernels: s[b][h][c] = state at the
 * start of 32-token chunk c, c < ceil(T/32), the rest of s and all of sa untouched; general-shape
 * kernels: transposed state at the end of every chunk_len tokens, and sa).  No counterpart in the
 * reference. */
int rwkvb200_wkv7_select_path(int path);
/* Form of the tensor-core RWKV-7 kernels: 0 = automatic (forward: the staged kernel, three warp groups on
 * consecutive chunks with inputs by TMA; backward: the two-stage kernel for launches with at most one
 * (batch, head) unit per SM, the one-group kernel otherwise), 1 = one-group kernels, 2 = staged / two-stage
 * kernels.  All run the same products; results agree to the last bf16 digit (a few dw elements differ by one ulp).
 * Process-wide; no counterpart in the reference. */
int rwkvb200_wkv7_select_form(int form);
/* Synchronous read of the current device's sticky status word: 0, or 10 + n / 20 + n when the n-th
 * bounded wait of the tensor-core forward / backward ran out in some thread block (30.. / 40..: the
 * front / back warp group of the two-stage backward, 50.. / 55.. / 60..: loader / matrix / chain group of the
 * staged forward; 70.. / 75.. / 80..: the same groups of the staged RWKV-6 / RWKV-5 forward; 91..: their tcgen05 backward) (the outputs of
 * that call are then invalid); negative on a CUDA error.  Per device; stays set until cleared. */
int rwkvb200_device_status(void);
/* Resets the current device's status word.  No counterpart in the reference. */
int rwkvb200_device_status_clear(void);
/* Test hook: the next tensor-core rwkvb200_wkv7_forward call does not issue the first product of its
 * first chunk and polls for it 2^10 times only, so that the bounded-wait path (status word, release of
 * tensor memory, orderly return) can be exercised with nothing in flight.  That call's outputs are
 * invalid.  No counterpart in the reference. */
int rwkvb200_wkv7_test_expire_next_forward(void);
/* Test hook: on != 0 makes the library behave as if the driver could not make tensor maps, so that the kernels that
 * load their inputs without TMA (the one-group RWKV-7 forward, the plain-load paths of the backward kernels, the
 * mma.sync RWKV-5/6 forward) run; 0 restores the normal choice.  Process-wide.  No counterpart in the reference. */
int rwkvb200_test_disable_tensor_maps(int on);

#ifdef __cplusplus
}
#endif
#endif /* RWKVB200_H */
