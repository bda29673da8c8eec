/*
 * kuiops.h -- C ABI of the B200 (sm_100a) kuiops operator library.
 *
 * The reference project (panther03/kuiLLM) has no fixed C ABI: every kernel
 * instantiation is extracted to a host launcher `<Module>_<name>(dims..., ptrs...)`
 * whose prototype sits in a generated `_decl.h` (kuipy/toolchain.py:171-182,
 * kuipy/compile.py:98-112) and is called from a per-family pybind wrapper
 * template (kuiops/<op>/wrapper_<op>.cu.j2).  This header fixes those launcher
 * calls as one stable set of `extern "C"` entry points.  Each declaration cites
 * the reference launcher call it replaces; the argument order of the reference
 * is kept (dims first, then pointers), followed by the additions every entry
 * point shares: caller-owned workspace where a kernel needs scratch, and the
 * CUDA stream.
 *
 * Conventions
 *   - Plain pointers and sizes only.  All pointers are device pointers unless a
 *     parameter is documented as a host array (shape vectors, pointer tables).
 *   - Every entry point returns KUIOPS_OK (0) or a negative KUIOPS_E* code.
 *     Contract violations are detected on the host and nothing is launched.
 *   - Nothing here allocates, frees or synchronises.  Work is enqueued on
 *     `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *   - Tensors are dense row-major unless a leading dimension is given.
 *   - Workspaces are handed over zero-filled once; a kernel that runs to completion
 *     leaves the ticket / counter words at the head of its workspace zero for the
 *     next call.  After any error (a negative return code, or a non-zero word from
 *     kuiops_debug_tc_error) the caller must zero the workspace again before
 *     reusing it: a kernel that gave up mid-way may have left counters non-zero.
 *   - `status` parameters are optional device int32 words.  A kernel that meets
 *     an out-of-range index skips that access and stores a non-zero code there.
 *   - The library is re-entrant.  The only process-wide state is the driver
 *     entry point used to encode TMA descriptors, resolved once under a mutex.
 */
#ifndef KUIOPS_H_
#define KUIOPS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KUIOPS_ABI_VERSION 1

/* ---- return codes ------------------------------------------------------- */
#define KUIOPS_OK             0
#define KUIOPS_EINVAL        (-1)  /* a shape/stride/dtype contract does not hold     */
#define KUIOPS_EUNSUPPORTED  (-2)  /* legal request outside what the kernels cover     */
#define KUIOPS_EWORKSPACE    (-3)  /* workspace missing or smaller than *_workspace_bytes */
#define KUIOPS_ELAUNCH       (-4)  /* the CUDA runtime refused the launch              */
#define KUIOPS_EDRIVER       (-5)  /* TMA descriptor encoding failed                   */
#define KUIOPS_ELIMIT        (-6)  /* size beyond a stated fixed maximum               */

/* ---- element types ------------------------------------------------------ */
#define KUIOPS_F32   0
#define KUIOPS_BF16  1
#define KUIOPS_F16   2

typedef void* kuiops_stream_t;

#if defined(__GNUC__)
#define KUIOPS_API __attribute__((visibility("default")))
#else
#define KUIOPS_API
#endif

KUIOPS_API int         kuiops_abi_version(void);
KUIOPS_API const char* kuiops_strerror(int code);
/* Diagnostics for the tensor-core kernels, whose pipeline waits are bounded: copies the
 * device-side error word to *host_out (0 = no wait ever ran out; otherwise the code of the
 * wait that gave up) and optionally clears it.  Synchronises the device. */
KUIOPS_API int kuiops_debug_tc_error(unsigned int* host_out, int reset);
/* Self-timing of the tcgen05 GEMM: while `device_buffer` (>= 32 uint64 on the current device) is set,
 * CTA 0 of every GEMM launched afterwards stores the global nanosecond timer at the stations of its
 * critical path: [0] CTA start, [1] predecessor kernel complete, [2] first operand tiles landed,
 * [3] last MMA issued, [4] accumulator complete, [5] split-K partial parked, [6] cluster met,
 * [7] tile share reduced and stored (with the push epilogue: sent), [8] cluster met again.
 * kuiops_rmsnorm_gather stamps [12] CTA start, [13] predecessor complete, [14] its cells of every rank
 * seen, [15] rows stored.  The split-KV decode attention stamps [16] CTA start, [17] predecessor
 * complete, [18] first scores ready, [19] all tiles accumulated, [20] record parked, [21] merged (by
 * the last slice), [22] epilogue done.  NULL switches it off (the default).
 * No counterpart in the reference. */
KUIOPS_API int kuiops_debug_gemm_trace(uint64_t* device_buffer);
/* How long kuiops_rmsnorm_gather polls for a peer's cells before it gives up, stores
 * error word 30 (see kuiops_debug_tc_error), sums whatever the receive slots hold and returns.
 * Nanoseconds; 0 restores the default of two seconds.  Returns the previous value.  A peer that
 * died between steps therefore costs one limit per launch instead of a hang; tests use a
 * millisecond limit with cells nobody stamps.  No counterpart in the reference (it has no
 * multi-GPU path). */
KUIOPS_API uint64_t kuiops_debug_set_peer_wait_ns(uint64_t ns);
/* Programmatic dependent launch for the short kernels of a decode step (GEMM, attention,
 * RMSNorm, RoPE, SwiGLU, embedding, arg-max): when enabled (default; KUIOPS_PDL=0 in the
 * environment or a 0 here turns it off) they are launched so that their set-up overlaps the
 * tail of the previous kernel in the stream; each waits for that kernel's completion before
 * touching memory, so results do not change.  Returns the previous setting. */
KUIOPS_API int kuiops_set_pdl(int enabled);
/* Number of kernels this library has enqueued since load (all threads). */
KUIOPS_API uint64_t    kuiops_launch_count(void);

/* ======================================================================== */
/* GEMM family                                                              */
/* ======================================================================== */

/* General entry every GEMM-shaped op lowers to.
 *   C[b] = alpha * A[b] x B[b] + beta * Cin[b]          (b = 0..batch-1)
 * A is [M,K] with leading dimension lda.  B is [K,N] with leading dimension ldb
 * when trans_b == 0, or is stored as [N,K] (the `weight.t()` view of a Linear
 * layer) with leading dimension ldb when trans_b == 1.  Cin may be NULL (beta is
 * then ignored); ldcin == 0 means Cin is a length-N row vector broadcast over
 * rows (the fused bias of addmm).  Inputs are `dtype`; C is `out_dtype`
 * (same as dtype, or KUIOPS_F32).  Accumulation is always fp32.
 * bf16/f16 operands whose pointers are 16-byte aligned and whose leading
 * dimensions are multiples of 8 run on the tcgen05 tensor-core kernels; M <= 128
 * uses the weight-streaming placement, which splits K over the CTAs of a
 * thread-block cluster and reduces the partials in shared memory (in-kernel,
 * deterministic).  Everything else (fp32, odd strides) runs on the SIMT kernel.
 * `workspace` is reserved: the current kernels keep their partials on chip and
 * ignore it (NULL is accepted); kuiops_gemm_workspace_bytes reports the size a
 * caller should provide to stay compatible with kernels that may use it.
 * Replaces the launchers at wrapper_mm.cu.j2:15-19, wrapper_addmm.cu.j2:18-24
 * and wrapper_bmm.cu.j2:16-20. */
#define KUIOPS_GEMM_COUNTER_BYTES 16384
KUIOPS_API size_t kuiops_gemm_workspace_bytes(int dtype, uint32_t batch, uint32_t M, uint32_t N, uint32_t K);

/* Tuned plans of the tcgen05 GEMM.  The kernel chooses its K split (weight-streaming placement,
 * M <= 128: 1..8 CTAs of a cluster share a tile) and its column tile (normal placement: 128 or
 * 256) by rule; a tuner that has timed the alternatives of a shape records its choice here and
 * every later call of that shape (batch 1) uses it.  `epilogue`: 0 plain / bias, 1 SwiGLU, 2 rotary.
 * splits == 0 keeps the rule for the split, bn == 0 for the tile; both 0 forgets the shape.
 * Results do not depend on the column tile; a different K split changes the order of the fp32
 * partial sums (still deterministic for a given plan).  kuiops_gemm_tune_query reports the plan a
 * shape would run with.  Host-side table, process wide, guarded by a mutex.
 * Reference: the per-family tune_params hook, kuipy/kuiops.py:27-43 and kuipy/registry.py:62-76
 * (load / save are stubs there; its tile choosers pick the first fitting tile, kuiops.py:330-394). */
KUIOPS_API int kuiops_gemm_tune_set(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K,
                                    int splits, int bn);
KUIOPS_API int kuiops_gemm_tune_clear(void);
KUIOPS_API int kuiops_gemm_tune_query(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K,
                                      int* splits, int* bn, int* swapped);
/* Number of SMs (0..64, default 0) the persistent GEMM (M > 128: one CTA per SM) leaves free from now on, process
 * wide; returns the previous value.  For hosts that run a communication kernel on another stream beside the GEMMs
 * (the tensor-parallel prefill sums one half-batch's partial products while the other half computes): a persistent
 * grid that fills every SM makes such a kernel wait for the GEMM to end.  Results do not depend on it.  No
 * counterpart in the reference (single GPU, kuipy/kuiops.py:397-469). */
KUIOPS_API int kuiops_gemm_set_sm_reserve(int sms);
KUIOPS_API int kuiops_gemm(int dtype, int out_dtype, uint32_t batch,
                uint32_t M, uint32_t N, uint32_t K,
                const void* A, int64_t lda, int64_t stride_a,
                const void* B, int64_t ldb, int64_t stride_b, int trans_b,
                const void* Cin, int64_t ldcin, int64_t stride_cin,
                float alpha, float beta,
                void* C, int64_t ldc, int64_t stride_c,
                void* workspace, size_t workspace_bytes,
                kuiops_stream_t stream);

/* Fused MLP front half: Y[m, j] = silu(A w_gate_j) * (A w_up_j), one tensor-core GEMM whose
 * epilogue applies the activation, so the [M, 2N] gate|up product never reaches memory.
 * W is [2N, K] (leading dimension ldw) with gate and up rows interleaved: row 2j = w_gate_j,
 * row 2j + 1 = w_up_j.  bf16 / f16 operands that meet the tensor-core alignment rules only
 * (KUIOPS_EUNSUPPORTED otherwise: run kuiops_gemm then kuiops_swiglu).  The dispatcher sees this
 * as mm, mm, silu, mul (kuipy/kuiops.py:158,166 of the reference); no reference counterpart. */
KUIOPS_API int kuiops_gemm_swiglu(int dtype, uint32_t M, uint32_t N, uint32_t K,
                const void* A, int64_t lda, const void* W, int64_t ldw, void* Y, int64_t ldy,
                void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

/* Packed QKV projection of a decode-sized step with the rotary embedding and the KV-cache append
 * in its epilogue: qkv[m, :] = A[m, :] x W^T with W = [(hq + 2 hk) * 128, K] (q heads, then k heads,
 * then v heads, head dimension 128); q and k heads get the rotary embedding of positions[m]
 * (rotate-half convention, base theta), and k / v heads are also written to
 * k_cache / v_cache[(m / rows_per_seq), kv head, positions[m], :] (capacity cache_cap rows per
 * sequence; the caches may be NULL).  Results are bit for bit those of kuiops_gemm followed by
 * kuiops_rope_qkv.  bf16 / f16, M <= 128, tensor-core alignment rules, and K large enough for the
 * split-K placement (KUIOPS_EUNSUPPORTED otherwise: run the two calls).  The dispatcher sees this
 * as mm, mul, cat, neg, add (kuipy/kuiops.py:158-166 of the reference); no reference counterpart. */
KUIOPS_API int kuiops_gemm_rope_qkv(int dtype, uint32_t M, uint32_t hq, uint32_t hk, uint32_t d, uint32_t K,
                const void* A, int64_t lda, const void* W, int64_t ldw, void* qkv, int64_t ldq,
                const int64_t* positions, float theta, void* k_cache, void* v_cache, uint64_t cache_cap,
                uint32_t rows_per_seq, kuiops_stream_t stream);

/* RMSNorm folded into the two GEMMs around it (decode-sized steps, M <= 128, bf16 / f16, weights [N, K]).
 * In a decoder layer  r' = r + A W^T ;  h = rmsnorm(r') * g ;  y = h V^T  costs three launches.  Folded:
 *   kuiops_gemm_residual_ssq:  resid[m, :] += A[m, :] W^T in place (one rounding), and
 *       ssq_out[t * M + m] = sum over the 128 features n of tile t of resid[m, n]^2 as stored
 *       (t < ceil(N / 128); fp32; every entry is written, no zeroing needed);
 *   kuiops_gemm_swiglu_rms / kuiops_gemm_rope_qkv_rms: kuiops_gemm_swiglu / kuiops_gemm_rope_qkv on the
 *       UN-normalised rows A = resid, with row m of the product multiplied by
 *       rsqrt(sum_t ssq[t * M + m] / K + eps) before the epilogue.  The norm weight g must have been
 *       multiplied into the columns of V beforehand (V'[n, k] = V[n, k] * g[k]).
 * The partials are summed per row in tile order, so the result is deterministic.  Against the
 * three-launch form the normalised rows are no longer rounded to the element type before the
 * product (results agree within the bf16 bar, not bit for bit).  KUIOPS_EUNSUPPORTED for shapes
 * outside the weight-streaming placement: run the unfused calls.  The dispatcher sees this as
 * add, pow, mean, add, rsqrt, mul, mul, mm (kuipy/kuiops.py:116-121,397-469 of the reference); no
 * reference counterpart. */
KUIOPS_API int kuiops_gemm_residual_ssq(int dtype, uint32_t M, uint32_t N, uint32_t K,
                const void* A, int64_t lda, const void* W, int64_t ldw,
                void* resid, int64_t ldr, float* ssq_out, kuiops_stream_t stream);
KUIOPS_API int kuiops_gemm_swiglu_rms(int dtype, uint32_t M, uint32_t N, uint32_t K,
                const void* A, int64_t lda, const void* W, int64_t ldw, void* Y, int64_t ldy,
                const float* ssq, uint32_t ssq_tiles, float eps, kuiops_stream_t stream);
KUIOPS_API int kuiops_gemm_rope_qkv_rms(int dtype, uint32_t M, uint32_t hq, uint32_t hk, uint32_t d, uint32_t K,
                const void* A, int64_t lda, const void* W, int64_t ldw, void* qkv, int64_t ldq,
                const int64_t* positions, float theta, void* k_cache, void* v_cache, uint64_t cache_cap,
                uint32_t rows_per_seq, const float* ssq, uint32_t ssq_tiles, float eps, kuiops_stream_t stream);

/* Tensor-parallel row-split GEMM fused with the first half of its all-reduce (decode shapes,
 * M <= 128, N a multiple of 4, bf16 / f16): rank `rank` of `n_ranks` computes its partial product
 * A x B (B as in kuiops_gemm: [K,N], or [N,K] when trans_b) and the epilogue stores it, through
 * peer pointers, into the receive area of EVERY rank (its own included) instead of a local C:
 *     peer_base[r] + ((epoch & 1) * n_ranks + rank) * slot_bytes
 * as M x N / 2 cells of 8 bytes, row-major: two consecutive elements of a row (4 bytes) and the
 * 32-bit stamp epoch + 1.  A cell is valid for the consumer the moment it is seen with the
 * expected stamp, so the exchange needs no fence, no flag word and no completion step: latency is
 * one NVLink store.  slot_bytes >= 4 * M * N, a multiple of 16.  `peer_base` is a HOST array of
 * n_ranks device addresses: the same symmetric allocation as mapped into this process for each
 * rank (16-byte aligned, 2 * n_ranks * slot_bytes long, zero-filled once before the first
 * launch).  `epoch` is this rank's device word that kuiops_rmsnorm_gather advances after it has
 * consumed the partials.  Producer and consumer alternate on the stream, so two halves of slots
 * are enough: a rank cannot push epoch e + 2 before it has consumed e + 1, which every peer pushed
 * only after consuming e; a cell left over from epoch e carries the stamp e + 1 and is never taken
 * for one of epoch e + 2.
 * The collective is plain peer stores over NVLink; no library call, no multicast.
 * No counterpart in the reference (it has no multi-GPU path); the single-rank form is
 * wrapper_mm.cu.j2:15-19. */
#define KUIOPS_MAX_PEERS 8
KUIOPS_API int kuiops_gemm_push(int dtype, uint32_t M, uint32_t N, uint32_t K,
                const void* A, int64_t lda, const void* B, int64_t ldb, int trans_b,
                uint32_t n_ranks, uint32_t rank, const uint64_t* peer_base,
                uint64_t slot_bytes, const uint32_t* epoch, kuiops_stream_t stream);

/* Second half of that all-reduce, fused with the residual add and the RMSNorm that follow a
 * row-split projection in a decoder layer: every thread polls the cells it is about to sum in the
 * slots of all `n_ranks` ranks until they carry the stamp of the current epoch (bounded: about
 * 2 s unless lowered with kuiops_debug_set_peer_wait_ns; on expiry the error word read by
 * kuiops_debug_tc_error is set to 30 and the kernel continues with what it has), then
 *        x = sum_r slot(epoch & 1, r)   (fp32, rank order, rounded to dtype),
 *        residual_out = x + residual,   y = rmsnorm(residual_out) * weight,
 * and advances `epoch` by one.  `recv_base` is this rank's own receive area (peer_base[rank] of
 * kuiops_gemm_push), `ticket` a zeroed device word the kernel leaves zero.  bf16 / f16.
 * No counterpart in the reference. */
KUIOPS_API int kuiops_rmsnorm_gather(int dtype, uint64_t m, uint32_t n, uint32_t n_ranks,
                const void* recv_base, uint64_t slot_bytes,
                uint32_t* epoch, uint32_t* ticket,
                const void* residual, const void* weight, float eps,
                void* y, void* residual_out, kuiops_stream_t stream);

/* aten.mm: C[M,N] = A[M,K] x B[K,N], all dense row-major.
 * Reference launcher: (u32 M, u32 N, u32 K, in* A, in* B, out* C), kuiops/mm/wrapper_mm.cu.j2:15-19.
 * The reference's bf16 kernel writes fp32 and the Python side casts
 * (kuipy/kuiops.py:428,467-468); here C has the input dtype. */
KUIOPS_API int kuiops_mm_f32 (uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, void* C,
                   void* workspace, size_t workspace_bytes, kuiops_stream_t stream);
KUIOPS_API int kuiops_mm_bf16(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, void* C,
                   void* workspace, size_t workspace_bytes, kuiops_stream_t stream);
KUIOPS_API int kuiops_mm_f16 (uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, void* C,
                   void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

/* aten.addmm with a full [M,N] C: C := beta*C + alpha*(A x B), in place on C
 * (the caller passes a clone of the bias matrix, as the reference wrapper does).
 * Reference launcher: (u32 M, u32 K, u32 N, et alpha, et beta, A, B, C) -- note
 * the M,K,N order -- kuiops/addmm/wrapper_addmm.cu.j2:18-24. */
KUIOPS_API int kuiops_addmm_f32 (uint32_t M, uint32_t K, uint32_t N, float alpha, float beta,
                      const void* A, const void* B, void* C,
                      void* workspace, size_t workspace_bytes, kuiops_stream_t stream);
KUIOPS_API int kuiops_addmm_bf16(uint32_t M, uint32_t K, uint32_t N, float alpha, float beta,
                      const void* A, const void* B, void* C,
                      void* workspace, size_t workspace_bytes, kuiops_stream_t stream);
KUIOPS_API int kuiops_addmm_f16 (uint32_t M, uint32_t K, uint32_t N, float alpha, float beta,
                      const void* A, const void* B, void* C,
                      void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

/* aten.bmm: C[b] = A[b] x B[b].  Reference launcher: (u32 B, u32 M, u32 K, u32 N, A, B, C),
 * kuiops/bmm/wrapper_bmm.cu.j2:16-20. */
KUIOPS_API int kuiops_bmm_f32 (uint32_t batch, uint32_t M, uint32_t K, uint32_t N,
                    const void* A, const void* B, void* C,
                    void* workspace, size_t workspace_bytes, kuiops_stream_t stream);
KUIOPS_API int kuiops_bmm_bf16(uint32_t batch, uint32_t M, uint32_t K, uint32_t N,
                    const void* A, const void* B, void* C,
                    void* workspace, size_t workspace_bytes, kuiops_stream_t stream);
KUIOPS_API int kuiops_bmm_f16 (uint32_t batch, uint32_t M, uint32_t K, uint32_t N,
                    const void* A, const void* B, void* C,
                    void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

/* ======================================================================== */
/* Scaled dot-product attention                                             */
/* ======================================================================== */

/* out = softmax(scale * Q K^T [+ bias] [causal mask]) V and the natural-log
 * row log-sum-exp.  Q is (n, h, l, e), K is (n, h_kv, s, e), V is (n, h_kv, s, ev),
 * out is (n, h, l, ev), lse (optional, fp32) is (n, h, l).  h must be a multiple
 * of h_kv (grouped-query attention: query head i reads KV head i / (h / h_kv)).
 * Strides are in elements for dims (batch, head, row); the innermost dim is
 * contiguous.  `bias` (optional, same dtype, dense (n, h, l, s)) is added to the
 * scaled scores as aten does.  With is_causal, query row i sees keys
 * j <= i + (s - l) (bottom-right aligned, so decode with l == 1 sees the whole
 * cache).  Reference launcher: (u32 n,h,l,s,e,ev, Q,K,V,bias, scale) returning
 * kernel-allocated out/lse, kuiops/sdpa/wrapper_sdpa.cu.j2:21-27; extended with
 * h_kv, is_causal, strides and caller-owned outputs.
 * bf16/f16 with e == ev == 128, no bias and l >= 64 run on the tcgen05 flash
 * kernel; short-query calls (l <= 16 with at most 128 query rows per KV head:
 * decode) run on the tcgen05 split-KV kernel, which spreads the keys of a
 * (batch, KV head) over several CTAs when there are few such pairs and then
 * needs kuiops_sdpa_workspace_bytes(...) of zero-initialised workspace (the query
 * returns 0 when no split is planned); everything else (bias, other head
 * dimensions, fp32) uses the generic SIMT kernel. */
KUIOPS_API size_t kuiops_sdpa_workspace_bytes(int dtype, uint32_t n, uint32_t h, uint32_t h_kv,
                                   uint32_t l, uint32_t s, uint32_t e, uint32_t ev);
KUIOPS_API int kuiops_sdpa(int dtype, uint32_t n, uint32_t h, uint32_t h_kv,
                uint32_t l, uint32_t s, uint32_t e, uint32_t ev,
                const void* Q, int64_t q_sn, int64_t q_sh, int64_t q_sl,
                const void* K, int64_t k_sn, int64_t k_sh, int64_t k_ss,
                const void* V, int64_t v_sn, int64_t v_sh, int64_t v_ss,
                const void* bias, float scale, int is_causal,
                void* out, int64_t o_sn, int64_t o_sh, int64_t o_sl,
                float* lse,
                void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

/* Same, with the number of keys of each batch entry read from device memory:
 * kv_lens[b] (int64, clamped to [0, s]) replaces s for entry b, s stays the
 * upper bound (the cache capacity in use).  A decode step whose launch
 * arguments never change can then be captured once in a CUDA graph and replayed
 * while the cache grows.  kv_lens == NULL is kuiops_sdpa.  Runs on the split-KV
 * kernels (tcgen05 where the shape allows, SIMT otherwise), never on the flash
 * kernel.  No counterpart in the reference. */
KUIOPS_API int kuiops_sdpa_varlen(int dtype, uint32_t n, uint32_t h, uint32_t h_kv,
                uint32_t l, uint32_t s, uint32_t e, uint32_t ev,
                const void* Q, int64_t q_sn, int64_t q_sh, int64_t q_sl,
                const void* K, int64_t k_sn, int64_t k_sh, int64_t k_ss,
                const void* V, int64_t v_sn, int64_t v_sh, int64_t v_ss,
                const void* bias, float scale, int is_causal,
                void* out, int64_t o_sn, int64_t o_sh, int64_t o_sl,
                float* lse, const int64_t* kv_lens,
                void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

/* Debug: force the number of key slices of the split-KV decode kernel (0 restores its rule); the
 * workspace query follows the override.  Used to sweep the split count of a shape.  No counterpart
 * in the reference. */
KUIOPS_API int kuiops_debug_sdpa_splits(int splits);

/* Attention for callers that must not allocate device memory.
 * Has no counterpart in the reference.
 * Some hosts of this library cannot call cudaMalloc around an attention call: a
 * plugin loaded into another runtime that has already claimed the whole device
 * for its own pool, or a serving loop that may not take the device-wide stall an
 * allocation can cause.  kuiops_sdpa leaves the split-KV scratch to the caller;
 * this variant needs none: the partial (max, sum, output) records of the split
 * keys go to a fixed array of KUIOPS_SDPA_NOALLOC_SCRATCH_BYTES that is part of
 * the library image (each GPU that loads the library holds one copy until the
 * process exits).  Inputs and outputs are still the caller's.  Arguments and
 * results are those of kuiops_sdpa_varlen (kv_lens may be NULL).
 *   - A problem whose scratch need exceeds the array is refused with
 *     KUIOPS_ELIMIT; nothing is launched.  The need is that of the kernel these
 *     arguments select (never more than kuiops_sdpa_workspace_bytes reports).
 *   - The array used is the copy on the GPU that holds Q, whichever device the
 *     calling thread has current; `stream` must belong to that GPU.  The first
 *     call for a GPU looks up the array's address there; make that first call
 *     before starting any stream capture.
 *   - All calls share the one array and it keeps the last call's contents; the
 *     entry point clears the ticket words it relies on, on `stream`, before the
 *     kernel.  Two calls that overlap on the GPU (different streams) race on it:
 *     serialise them.
 *   - No cudaMalloc, cudaFree or allocating library routine is called. */
#define KUIOPS_SDPA_NOALLOC_SCRATCH_BYTES (8u << 20)
KUIOPS_API int kuiops_sdpa_noalloc(int dtype, uint32_t n, uint32_t h, uint32_t h_kv,
                uint32_t l, uint32_t s, uint32_t e, uint32_t ev,
                const void* Q, int64_t q_sn, int64_t q_sh, int64_t q_sl,
                const void* K, int64_t k_sn, int64_t k_sh, int64_t k_ss,
                const void* V, int64_t v_sn, int64_t v_sh, int64_t v_ss,
                const void* bias, float scale, int is_causal,
                void* out, int64_t o_sn, int64_t o_sh, int64_t o_sl,
                float* lse, const int64_t* kv_lens, kuiops_stream_t stream);

/* ======================================================================== */
/* Streaming reductions                                                     */
/* ======================================================================== */

/* Row softmax of an [m, n] row-major matrix over n.  Y may equal X (the
 * reference kernel is in place on the caller's clone).
 * Reference launcher: (u32 m, u32 n, T* X), kuiops/softmax/wrapper_softmax.cu.j2:14-16. */
KUIOPS_API int kuiops_softmax_f32 (uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t stream);
KUIOPS_API int kuiops_softmax_bf16(uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t stream);
KUIOPS_API int kuiops_softmax_f16 (uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t stream);

/* Last-axis mean with keepdim: out[i] = sum_j in[i,j] / n, fp32 accumulation.
 * Reference launcher: (size_t m, size_t n, in*, out*), kuiops/mean/wrapper_mean.cu.j2:28-31. */
KUIOPS_API int kuiops_mean_f32 (uint64_t m, uint64_t n, const void* in, void* out, kuiops_stream_t stream);
KUIOPS_API int kuiops_mean_bf16(uint64_t m, uint64_t n, const void* in, void* out, kuiops_stream_t stream);
KUIOPS_API int kuiops_mean_f16 (uint64_t m, uint64_t n, const void* in, void* out, kuiops_stream_t stream);

/* Categorical sampling: out[i, j] = an index of row i of the [m, n] fp32 weight matrix drawn with
 * probability weights[i, k] / sum_k weights[i, k], num_samples draws per row, independent (with
 * replacement).  aten.multinomial(probs, num_samples, replacement) for num_samples == 1 or
 * replacement == True.  No counterpart in the reference beyond the backlog entry (KERNELS.md:68-90).
 * The random stream is documented so that every draw can be recomputed: u(i, j) = (x0 >> 8) * 2^-24
 * with (x0, ..) = Philox4x32-10(counter = (offset low, offset high, i, j), key = (seed low, seed
 * high)), and the index is found by inverting the row's running fp32 sum evaluated in a fixed
 * order (see csrc/sampling.cu); an element of weight zero is never drawn.  PyTorch's own draws use
 * a stream private to its kernels, so results agree in distribution, not bit for bit.  A negative,
 * infinite or NaN weight counts as zero and stores 2 in *status; a row without any weight yields
 * index 0 and stores 3 (`status` may be NULL). */
KUIOPS_API int kuiops_multinomial_f32(uint32_t m, uint32_t n, uint32_t num_samples, const void* weights, int64_t* out,
                                      uint64_t seed, uint64_t offset, int* status, kuiops_stream_t stream);

/* One token per row of an [m, n] fp32 logit matrix: temperature, top-k filter, top-p (nucleus) filter and the
 * draw in two launches that read the logits once (the selection's second look comes from L2), instead of the
 * separate div / topk / sort / softmax / cumsum / scatter / multinomial calls a sampling loop makes
 * (infer.py:139-143 samples with temperature 0.7 through HuggingFace's warpers).  No counterpart in the
 * reference.  The set kept is the one those warpers keep: the top_k largest logits (equal values: lowest index
 * first), weights e_r = exp((v_r - v_max) / temperature) taken largest first, rank r kept while the running sum
 * before it is below top_p times the sum of all top_k weights (rank 0 always).  The draw is
 * u = (x0 >> 8) * 2^-24, (x0, ..) = Philox4x32-10(counter = (offset low, offset high, row, 0), key = (seed low,
 * seed high)); the token is the first kept rank whose running sum exceeds u times the kept sum (running sums in
 * the fixed order csrc/sampling.cu states).  out[row] = the token id; out_prob (nullable) [m] fp32 = its
 * probability under the filtered distribution.  temperature > 0, 0 < top_p <= 1, 1 <= top_k (min(top_k, n)
 * <= 1024, else KUIOPS_ELIMIT).  workspace: kuiops_sample_workspace_bytes(m, min(top_k, n)) bytes, 16-byte
 * aligned, no initial contents required. */
KUIOPS_API size_t kuiops_sample_workspace_bytes(uint32_t m, uint32_t top_k);
KUIOPS_API int kuiops_sample_topk_topp_f32(uint32_t m, uint32_t n, const void* logits, float temperature, uint32_t top_k,
                                           float top_p, uint64_t seed, uint64_t offset, int64_t* out, float* out_prob,
                                           void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

/* Whole-tensor folds to one device scalar (aten.all / aten.any over bool bytes,
 * aten.max over int64 / fp32).  Reference: Kuiops.HReducePoly.Exact.reduce,
 * kuiops/reduce/Kuiops.HReducePoly.Exact.fsti:26-46 (which mallocs the result
 * and copies it to the host, .fst:1029-1036; here the scalar stays on the
 * device at `out`).  workspace: KUIOPS_REDUCE_WORKSPACE_BYTES, first 8 bytes
 * zero on first use and left zero. */
#define KUIOPS_REDUCE_ALL 0
#define KUIOPS_REDUCE_ANY 1
#define KUIOPS_REDUCE_MAX 2
#define KUIOPS_REDUCE_WORKSPACE_BYTES 16384
KUIOPS_API int kuiops_reduce_u8 (int op, uint64_t n, const void* in, void* out,
                      void* workspace, size_t workspace_bytes, kuiops_stream_t stream);
KUIOPS_API int kuiops_reduce_i64(int op, uint64_t n, const void* in, void* out,
                      void* workspace, size_t workspace_bytes, kuiops_stream_t stream);
KUIOPS_API int kuiops_reduce_f32(int op, uint64_t n, const void* in, void* out,
                      void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

/* aten.topk over the last axis of an [m, n] fp32 matrix, largest first.
 * values is [m, k] fp32, indices [m, k] int64.  Equal values are ordered by
 * ascending index, and NaN sorts above +inf (torch's ordering).  k <= 2048.
 * No reference kernel exists (kuiops/topk/ is empty); signature from KERNELS.md:58. */
KUIOPS_API int kuiops_topk_f32(uint32_t m, uint32_t n, uint32_t k, const void* X,
                    void* values, int64_t* indices, kuiops_stream_t stream);

/* ======================================================================== */
/* Indexed data movement (payload moves: any element size 1, 2, 4, 8 bytes) */
/* ======================================================================== */
#define KUIOPS_MAX_RANK 8

/* aten.gather: out[x] = inp[x with x[dim] := idx[x]], out has idx's shape.
 * Contract (Kuiops.Common.fsti:34-38, Kuiops.Gather.fsti:31-33): equal ranks,
 * idx_shape[d] <= inp_shape[d] for every d != dim, n == numel(idx) > 0 and every
 * index value in [0, inp_shape[dim]).  The reference demands idx_shape <=
 * inp_shape on `dim` too (kuipy/kuiops.py:736); that extra limit is kept in the
 * Python gate, not here.  The int64 index is read directly (the reference
 * narrows it to u32 with a strided copy first, include/kuiops.h:28-36).
 * inp_shape / idx_shape are host arrays of `rank` entries.
 * Reference launcher: (u32 inp dims.., u32 idx dims.., T* inp, u32* idx, T* out, u32 n),
 * kuiops/gather/wrapper_gather.cu.j2:26-32. */
KUIOPS_API int kuiops_gather(uint32_t elem_bytes, uint32_t rank, uint32_t dim,
                  const uint64_t* inp_shape, const uint64_t* idx_shape,
                  const void* inp, const int64_t* idx, void* out, uint64_t n,
                  int32_t* status, kuiops_stream_t stream);

/* aten.scatter.src: out = self; out[i with i[dim] := idx[i]] = src[i] for every
 * cell i of src (src and idx share one shape <= self's shape pointwise).
 * If self_ != out the library first copies self_ into out (the reference wrapper
 * clones on the host side, wrapper_scatter.cu.j2:25).  Duplicate targets are a
 * contract violation the kernel cannot see (Kuiops.Scatter.fsti:36-41): one of
 * the writers wins, as in PyTorch.
 * Reference launcher: (u32 self dims.., u32 src dims.., T* src, u32* idx, T* out, u32 n),
 * kuiops/scatter/wrapper_scatter.cu.j2:30-36. */
KUIOPS_API int kuiops_scatter(uint32_t elem_bytes, uint32_t rank, uint32_t dim,
                   const uint64_t* self_shape, const uint64_t* src_shape,
                   const void* self_, const void* src, const int64_t* idx, void* out, uint64_t n,
                   int32_t* status, kuiops_stream_t stream);

/* aten.cat of two tensors that agree off `dim`.
 * Reference launcher: (u32 a dims.., u32 b_dim, T* A, T* B, T* out, u32 n),
 * kuiops/cat/wrapper_cat.cu.j2:28-34; n must equal numel(out). */
KUIOPS_API int kuiops_cat(uint32_t elem_bytes, uint32_t rank, uint32_t dim,
               const uint64_t* a_shape, uint64_t b_dim,
               const void* A, const void* B, void* out, uint64_t n,
               kuiops_stream_t stream);

/* N-ary cat: `count` tensors whose shapes equal `shape` except along `dim`,
 * where tensor t has dim_sizes[t] entries.  ptrs and dim_sizes are host arrays.
 * No reference counterpart (the reference kernel is binary only,
 * kuipy/kuiops.py:822). */
KUIOPS_API int kuiops_cat_n(uint32_t elem_bytes, uint32_t rank, uint32_t dim, uint32_t count,
                 const uint64_t* shape, const uint64_t* dim_sizes,
                 const void* const* ptrs, void* out, kuiops_stream_t stream);

/* aten.index.Tensor with `n_idx` int64 index tensors applied to the adjacent
 * dims [first_dim, first_dim + n_idx) of a dense `self`.  The index tensors are
 * already broadcast to one shape idx_shape[idx_rank]; idx_strides holds
 * n_idx * idx_rank element strides (0 on broadcast dims).  Output shape is
 * self_shape[:first_dim] + idx_shape + self_shape[first_dim + n_idx:].
 * Negative indices wrap once; out-of-range ones are skipped and flagged.
 * idx_ptrs is a host array of device pointers.  No reference kernel exists
 * (kuiops/index/ is empty); signature from KERNELS.md:67. */
KUIOPS_API int kuiops_index(uint32_t elem_bytes, uint32_t self_rank, const uint64_t* self_shape,
                 uint32_t first_dim, uint32_t n_idx, const int64_t* const* idx_ptrs,
                 uint32_t idx_rank, const uint64_t* idx_shape, const int64_t* idx_strides,
                 const void* self_, void* out, int32_t* status, kuiops_stream_t stream);

/* aten.isin(elements int64[n], test_elements int64[m]) -> bool bytes [n].
 * No reference kernel exists (kuiops/isin/ is empty); signature from KERNELS.md:56-57. */
KUIOPS_API int kuiops_isin_i64(uint64_t n, const int64_t* elements, uint64_t m, const int64_t* test_elements,
                    int invert, void* out, kuiops_stream_t stream);

/* ======================================================================== */
/* Elementwise maps                                                         */
/* ======================================================================== */
/* The reference bakes the lambda and its constants into each instantiation
 * (kuipy/kuiops.py:292-296); here `op` selects it and `c0`, `c1` carry the
 * constants.  Y may equal X (the reference kernels are in place on a clone).
 * Reference launchers, kuiops/elementwise/wrapper_elementwise.cu.j2:20-42:
 *   map(len, T*), map2(len, T*, T*), map_nip(len, Tin*, Tout*), map3(len, u8*, T*, T*, T*). */
#define KUIOPS_MAP_SILU     0
#define KUIOPS_MAP_NEG      1
#define KUIOPS_MAP_RSQRT    2
#define KUIOPS_MAP_COS      3
#define KUIOPS_MAP_SIN      4
#define KUIOPS_MAP_POW      5   /* x ** c0                    */
#define KUIOPS_MAP_SQUARE   6   /* x * x  (the x**2 special case, kuiops.py:270-273) */
#define KUIOPS_MAP_ADD      7   /* x + c1 * (y | c0)          */
#define KUIOPS_MAP_MUL      8   /* x * (y | c0)               */
#define KUIOPS_MAP_SUB      9   /* x - c1 * (y | c0)          */
#define KUIOPS_MAP_DIV     10   /* x / (y | c0)               */
#define KUIOPS_MAP_BNOT    11   /* bool bytes                 */
#define KUIOPS_MAP_BAND    12
#define KUIOPS_MAP_BOR     13
#define KUIOPS_MAP_EQ      14   /* x == c0 -> bool byte       */
#define KUIOPS_MAP_LE      15
#define KUIOPS_MAP_LT      16
#define KUIOPS_MAP_GELU    17   /* tanh-free erf GELU, for the GPT-2-shaped config */
/* Unary map, or binary with a scalar constant: Y[i] = op(X[i], c0, c1). */
KUIOPS_API int kuiops_map (int dtype, int op, uint64_t len, const void* X, void* Y, double c0, double c1,
                kuiops_stream_t stream);
/* x[i] += delta over int64, in place (aten.add.Tensor(T(1,int64), int), listed as not
 * connected in the reference's KERNELS.md:9; used for device-side position counters). */
KUIOPS_API int kuiops_add_i64(uint64_t len, int64_t* x, int64_t delta, kuiops_stream_t stream);
/* Binary same-shape map: Y[i] = op(X[i], B[i]); c1 is the `alpha` of add/sub. */
KUIOPS_API int kuiops_map2(int dtype, int op, uint64_t len, const void* X, const void* B, void* Y, double c1,
                kuiops_stream_t stream);
/* Bool-byte maps (bitwise_not / and / or).  B is ignored for BNOT. */
KUIOPS_API int kuiops_map_u8(int op, uint64_t len, const void* X, const void* B, void* Y,
                  kuiops_stream_t stream);
/* Scalar comparisons, float in -> bool byte out. */
KUIOPS_API int kuiops_map_nip(int dtype, int op, uint64_t len, const void* X, void* Y, double c0,
                   kuiops_stream_t stream);
/* where(cond, a, b) with payload elements of elem_bytes. */
KUIOPS_API int kuiops_map3(uint32_t elem_bytes, uint64_t len, const void* cond, const void* A, const void* B,
                void* Y, kuiops_stream_t stream);

/* ======================================================================== */
/* Fused decoder-layer helpers (compositions of the maps above that the      */
/* dispatcher sees as pow/mean/add/rsqrt/mul, silu/mul, mul/cat/neg/add)     */
/* ======================================================================== */

/* y = (x [+ residual]) * rsqrt(mean((x [+ residual])^2) + eps) * weight, rows of
 * length n.  When residual != NULL, the sum is also written to residual_out
 * (may alias residual).  fp32 statistics. */
KUIOPS_API int kuiops_rmsnorm(int dtype, uint64_t m, uint32_t n, const void* x, const void* residual,
                   const void* weight, float eps, void* y, void* residual_out,
                   kuiops_stream_t stream);
/* y[i, j] = silu(gu[i, j]) * gu[i, n + j] for a fused [m, 2n] gate|up matrix. */
KUIOPS_API int kuiops_swiglu(int dtype, uint64_t m, uint32_t n, const void* gate_up, void* y,
                  kuiops_stream_t stream);
/* Rotary embedding (rotate-half form) applied in place to q (rows, hq, d) and
 * k (rows, hk, d) slices of a packed qkv row of `row_stride` elements; positions
 * is int64 [rows]; theta is the base.  Also appends the rotated k and the raw v
 * of each row to a (batch, hk, cap, d) cache at slot positions[row] when
 * k_cache != NULL; rows_per_seq consecutive rows belong to one sequence. */
KUIOPS_API int kuiops_rope_qkv(int dtype, uint64_t rows, uint32_t hq, uint32_t hk, uint32_t d,
                    void* qkv, int64_t row_stride, const int64_t* positions, float theta,
                    void* k_cache, void* v_cache, uint64_t cache_cap, uint32_t rows_per_seq,
                    kuiops_stream_t stream);
/* Dtype cast of a dense buffer between the float types (aten._to_copy with a dtype change;
 * src == dst is aten.clone).  Rounds to nearest even, as the eager cast does.  The reference lists
 * these as backlog (KERNELS.md:46-48) and has no kernel: no counterpart. */
KUIOPS_API int kuiops_cast(int src_dtype, int dst_dtype, uint64_t len, const void* X, void* Y, kuiops_stream_t stream);

/* aten.masked_fill.Scalar on same-shape dense operands: Y[i] = mask[i] ? value : X[i], mask as
 * bool bytes, value rounded to dtype.  Backlog in the reference (KERNELS.md:68-90): no counterpart. */
KUIOPS_API int kuiops_masked_fill(int dtype, uint64_t len, const void* X, const void* mask, double value, void* Y,
                kuiops_stream_t stream);

/* out[r, :] = table[ids[r], :] (aten.embedding), row length `width` elements. */
KUIOPS_API int kuiops_embedding(uint32_t elem_bytes, uint64_t rows, uint64_t width, uint64_t vocab,
                     const void* table, const int64_t* ids, void* out, int32_t* status,
                     kuiops_stream_t stream);
/* Row arg-max of an [m, n] matrix (greedy sampling); ties -> lowest index. */
KUIOPS_API int kuiops_argmax(int dtype, uint64_t m, uint64_t n, const void* X, int64_t* out,
                  kuiops_stream_t stream);
/* Inclusive prefix sum along the rows of an [m, n] matrix (aten.cumsum over the last axis): the
 * position ids a decoder derives from its attention mask (int64, wraps like the eager sum) and the
 * cumulative probabilities of nucleus sampling (fp32).  m * n <= 2^31.  Backlog in the reference
 * (KERNELS.md:68-90): no counterpart. */
KUIOPS_API int kuiops_cumsum_f32(uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t stream);
KUIOPS_API int kuiops_cumsum_i64(uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t stream);

/* Stable sort of every row of an fp32 [m, n] matrix (aten.sort over the last axis): values and
 * the int64 permutation, ascending or descending (descending != 0).  Equal values keep their
 * original order, -0 equals +0, NaN is the largest value.  X and values must not overlap.
 * m * n <= 2^31; the workspace holds two (key, index) buffers.  Backlog in the reference
 * (KERNELS.md:68-90): no counterpart. */
KUIOPS_API size_t kuiops_sort_workspace_bytes(uint32_t m, uint32_t n);
KUIOPS_API int kuiops_sort_f32(uint32_t m, uint32_t n, int descending, const void* X, void* values,
                    int64_t* indices, void* workspace, size_t workspace_bytes, kuiops_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KUIOPS_H_ */
