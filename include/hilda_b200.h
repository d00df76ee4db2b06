/* C ABI of libhilda_b200.so: hand-written sm_100a CUDA kernels for the token-parallel operator
 * path of hilda-kernel (RMSNorm, FusedAddRMSNorm, RoPE, SwiGLU, CrossEntropy,
 * FusedLinearCrossEntropy, GRPO loss).
 *
 * The reference library has no native layer: each operator is a Python launcher around a Triton
 * kernel. Each entry point below replaces one such launcher; the reference function it stands in
 * for is cited by file:line (paths relative to triton-kernels/ in hilda-kernel).
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless stated otherwise; nothing is allocated inside the
 *    library: outputs and workspaces are supplied by the caller (sizes via *_workspace_bytes);
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, no host sync;
 *  - dtype enum: 0 = float32, 1 = bfloat16, 2 = float16;
 *  - return value: 0 on success, negative HILDA_ERR_* otherwise;
 *  - 16-byte aligned pointers and row lengths that are multiples of 16 bytes take the vectorised
 *    kernels; anything else takes a slower generic kernel with identical results.
 */
#ifndef HILDA_B200_H
#define HILDA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HILDA_OK 0
#define HILDA_ERR_DTYPE (-1)
#define HILDA_ERR_ALIGN (-2)
#define HILDA_ERR_SIZE (-3)
#define HILDA_ERR_CUDA (-4)
#define HILDA_ERR_NULL (-5)
#define HILDA_ERR_DEVICE (-6)
#define HILDA_ERR_ARG (-7)

#define HILDA_F32 0
#define HILDA_BF16 1
#define HILDA_F16 2

/* ---- RMSNorm ------------------------------------------------------------------------------ */
/* Replaces rms_norm_forward (kernels/rms_norm.py:261-306). x,y: [n_rows, n_cols] row-major in
 * `dtype`; w: [n_cols] in `w_dtype`; rstd: [n_rows] fp32 (the only saved statistic). */
int hilda_rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t n_rows, int64_t n_cols,
                       float eps, int dtype, int w_dtype, void* stream);

/* Replaces fused_add_rms_norm_forward (kernels/fused_add_rms_norm.py:172-188):
 * s = x + r (rounded to dtype), y = rmsnorm(s) * w. */
int hilda_fused_add_rms_norm_fwd(const void* x, const void* r, const void* w, void* y, void* s, float* rstd,
                                 int64_t n_rows, int64_t n_cols, float eps, int dtype, int w_dtype, void* stream);

/* Bytes of fp32 scratch hilda_norm_bwd needs (one partial dW row per CTA). */
int64_t hilda_norm_bwd_workspace_bytes(int64_t n_rows, int64_t n_cols, int dtype);

/* Replaces rms_norm_backward (kernels/rms_norm.py:309-359) and fused_add_rms_norm_backward
 * (kernels/fused_add_rms_norm.py:191-232). x is the saved input (RMSNorm) or the saved sum S
 * (FusedAddRMSNorm); dy and ds may each be null (treated as zeros); dx = norm_bwd(dy) + ds;
 * dw: [n_cols] in w_dtype, reduced in a fixed order (bit-reproducible). */
int hilda_norm_bwd(const void* dy, const void* ds, const void* x, const void* w, const float* rstd, void* dx,
                   void* dw, float* workspace, int64_t n_rows, int64_t n_cols, int dtype, int w_dtype,
                   void* stream);

/* Kernel behind hilda_norm_bwd for vectorisable shapes (no counterpart in the reference). 1
 * (default) = automatic: for 32-bit rows every CTA stages its rows through a ring of shared-memory
 * slots filled by bulk asynchronous copies when three or more slots fit; else, and for 16-bit rows
 * always, the register kernel (one row in flight per CTA) with a bulk L2 prefetch of the CTA's next
 * row, in a lean form when a 16-bit row fills the plan exactly; 0 = register kernel, no prefetch;
 * 2 / 3 = register kernel with the prefetch 1 / 2 rows ahead; 4 = ring whenever two slots fit. The
 * explicitly chosen kernels (0, 2, 3, 4) and, for 32-bit rows, the automatic choice give the same dX
 * and dW bit for bit; the lean 16-bit kernel of the automatic choice has a thread plan and a grid of
 * its own, so its sums are grouped differently (same values within rounding). Other values only query. Returns the previous choice; per host thread.
 * Environment: HILDA_NORM_RING. */
int hilda_norm_bwd_set_path(int path);

/* No counterpart in the reference. hilda_norm_bwd without the workspace argument, for hosts that
 * cannot supply one (a C/FFI caller with no allocator to borrow from, or a server whose memory was
 * all handed to its own pool at start-up and which must not call cudaMalloc afterwards). The dW
 * partial sums use a 16 MiB array inside the library, one copy per GPU that loads it; when the
 * default launch would need more partial rows than fit, fewer CTAs run (dX unchanged bit for bit, dW
 * equal within the rounding of another summation grouping); only n_cols * 4 bytes >
 * hilda_norm_bwd_noalloc_max_bytes() returns HILDA_ERR_SIZE. The first call on a device resolves
 * the array's address: make it before any stream capture. All calls share the array, so calls that
 * may overlap on the GPU race; keep them ordered. Allocates nothing. */
int64_t hilda_norm_bwd_noalloc_max_bytes(void);
int hilda_norm_bwd_noalloc(const void* dy, const void* ds, const void* x, const void* w, const float* rstd,
                           void* dx, void* dw, int64_t n_rows, int64_t n_cols, int dtype, int w_dtype,
                           void* stream);

/* ---- RoPE --------------------------------------------------------------------------------- */
/* Replaces rope_forward / rope_backward (kernels/rope.py:113-136, :139-172) for q and k in one
 * launch. Tensors are indexed (batch, head, seq, head_dim) with a contiguous last dim;
 * q_strides / k_strides hold six element strides: (b, h, s) of the input, then of the output.
 * q_out may equal q_in (in place). cos/sin: half-width tables [1 or bsz, seq, head_dim/2] in
 * cs_dtype, cos_stride_b = 0 for a batch-1 table. backward != 0 applies the transpose rotation
 * (-sin). Either tensor may be skipped with n_*_heads = 0. */
int hilda_rope(const void* q_in, void* q_out, const int64_t* q_strides, int n_q_heads, const void* k_in,
               void* k_out, const int64_t* k_strides, int n_k_heads, const void* cos, const void* sin,
               int64_t cos_stride_b, int64_t cos_stride_s, int bsz, int seq, int head_dim, int dtype,
               int cs_dtype, int backward, void* stream);

/* ---- SwiGLU ------------------------------------------------------------------------------- */
/* Replaces swiglu_forward (kernels/swiglu.py:112-124): c = silu(a) * b over n elements. */
int hilda_swiglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype, void* stream);
/* Replaces swiglu_backward (kernels/swiglu.py:127-141). da/db may alias a/b (the reference
 * overwrites the saved inputs). */
int hilda_swiglu_bwd(const void* a, const void* b, const void* dc, void* da, void* db, int64_t n, int dtype,
                     void* stream);

/* ---- GeGLU -------------------------------------------------------------------------------- */
/* Replace geglu_forward / geglu_backward (kernels/geglu.py:131-159): c = gelu_tanh(a) * b; the
 * backward may write da/db over a/b. */
int hilda_geglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype, void* stream);
int hilda_geglu_bwd(const void* a, const void* b, const void* dc, void* da, void* db, int64_t n, int dtype,
                    void* stream);

/* ---- CrossEntropy ------------------------------------------------------------------------- */
int64_t hilda_cross_entropy_workspace_bytes(int64_t n_rows);
/* Replaces cross_entropy_forward (kernels/cross_entropy.py:206-249). logits [n_rows, V] in dtype,
 * targets int64. grad != null: training path, grad = d loss / d logits for the given reduction
 * (0 none, 1 mean, 2 sum), written in the same pass; grad == null: inference path. loss_rows
 * [n_rows] fp32 (may be null -> kept in workspace), lse_rows optional, loss_out fp32 scalar for
 * mean/sum. Rows whose target equals ignore_index give loss 0 and a zero gradient row.
 * n_valid_in (nullable device int): number of valid rows to divide by for 'mean' instead of this
 * call's own count (row-sharded use: the count over all shards). */
int hilda_cross_entropy_fwd(const void* logits, const int64_t* targets, void* grad, float* loss_rows,
                            float* lse_rows, float* loss_out, void* workspace, const int* n_valid_in,
                            int64_t n_rows, int64_t V, int64_t ignore_index, int reduction, int dtype,
                            void* stream);

/* Replaces _ce_scale_grad_kernel (kernels/cross_entropy.py:173-189) and _element_mul_kernel
 * (kernels/fused_linear_cross_entropy.py:84-96): out = in * scale[0] or in[r,:] * scale[r];
 * scale is a device fp32 pointer; in and out may alias. */
int hilda_scale_rows(const void* in, void* out, const float* scale, int per_row, int64_t n_rows, int64_t n_cols,
                     int dtype, void* stream);

/* ---- FusedLinearCrossEntropy -------------------------------------------------------------- */
/* Replaces fused_linear_cross_entropy_forward (kernels/fused_linear_cross_entropy.py:103-171) on one
 * device: hidden [BT, H], W [V, H], targets [BT] int64; bf16 or fp16; H % 8 == 0. reduction 0
 * none (per-row loss in loss_rows), 1 mean, 2 sum (fp32 scalar loss_out). dh [BT, H] and dw [V, H]
 * (both or neither) receive the gradients for a unit upstream gradient. Rows are processed in
 * chunks of chunk_rows (<= 0: library default, scratch <= 1.25 GiB); the chunk's logits live in the
 * workspace, the full [BT, V] logits never exist. flags: HILDA_FLCE_COMPACT = the rows whose target
 * is ignore_index are compacted away ON THE DEVICE before the GEMMs (they contribute nothing to the
 * loss or to either gradient; their dh rows come back as zeros); the reference runs its GEMMs over
 * them and pays a host synchronisation for their count (:121), this call pays none. The call only
 * enqueues work; afterwards the int at workspace[0] is non-zero if a bounded device-side wait ran
 * out (HILDA_ERR_DEVICE), and a mean / sum loss is then NaN. */
#define HILDA_FLCE_COMPACT 1
int64_t hilda_flce_default_chunk_rows(int64_t BT, int64_t H, int64_t V);
int64_t hilda_flce_workspace_bytes(int64_t BT, int64_t H, int64_t V, int64_t chunk_rows, int with_grad, int flags);
int hilda_fused_linear_cross_entropy_fwd(const void* hidden, const void* W, const int64_t* targets, float* loss_out,
                                         float* loss_rows, void* dh, void* dw, void* workspace, int64_t BT,
                                         int64_t H, int64_t V, int64_t ignore_index, int reduction,
                                         int64_t chunk_rows, int dtype, int flags, void* stream);

/* The same operator as separate steps, for the vocab-parallel form (W sharded by rows over
 * ranks; no counterpart in the reference, which is single-device): between row_stats and
 * finalize the caller gathers the per-row (max, sum-exp, target logit) triples of all ranks.
 *   logits scratch: [hilda_flce_padded_rows(rows), hilda_flce_logits_pitch(V)] 16-bit
 *   stats:          [rows, hilda_flce_stat_tiles(V), 2] fp32
 *   rowstat:        [3, rows] fp32 = natural-log max, sum exp(x - max), target logit (0 if the
 *                   target is outside [vocab_start, vocab_start + V))
 * dyn_rows / dyn_off (dyn_rows nullable = off): a DEVICE int holding how many leading rows of the
 * whole (compacted) batch are real, and the index of this call's first row in that batch. Rows at
 * or beyond the count are skipped: GEMM tiles (logits, d hidden) and k-blocks (d W) beyond it do
 * not run. Their targets must equal ignore_index and their hidden rows must be zero up to the next
 * multiple of 256 (what hilda_flce_compact / hilda_gather_valid_rows produce). */
int64_t hilda_flce_logits_pitch(int64_t V);
int64_t hilda_flce_padded_rows(int64_t rows);
int64_t hilda_flce_stat_tiles(int64_t V);
/* *out = number of targets != ignore_index (kernels/fused_linear_cross_entropy.py:121, on device). */
int hilda_count_valid(const int64_t* targets, int64_t n, int64_t ignore_index, int* out, void* stream);
/* logits = hidden @ W^T rounded to dtype (fused_linear_cross_entropy.py:140) + online-LSE tile stats. */
int hilda_flce_logits(const void* hidden, const void* W, void* logits, float* stats, int64_t rows, int64_t H,
                      int64_t V, int dtype, int* status, const int* dyn_rows, int64_t dyn_off, void* stream);
/* The same with the statistics taken of logits * inv_temperature (stored logits unscaled): the
 * log-softmax at a temperature of the fused linear + JSD loss (kernels/fused_linear_jsd.py:46-62). */
int hilda_flce_logits_scaled(const void* hidden, const void* W, void* logits, float* stats, int64_t rows, int64_t H,
                             int64_t V, float inv_temperature, int dtype, int* status, void* stream);
/* targets may be null: no target logit is fetched (rowstat[2] = 0). */
int hilda_flce_row_stats(const float* stats, const void* logits, const int64_t* targets, float* rowstat,
                         int64_t rows, int64_t V, int64_t vocab_start, int dtype, const int* dyn_rows,
                         int64_t dyn_off, void* stream);
/* lse = max + log(sum-exp), loss = lse - target logit (0 on ignored rows). rowstat is [3, rows]
 * (n_shards <= 1) or the gathered [n_shards, 3, rows] of all vocabulary shards, merged here. */
int hilda_flce_finalize(const float* rowstat, int n_shards, const int64_t* targets, int64_t ignore_index,
                        float* lse, float* loss_rows, int64_t rows, const int* dyn_rows, int64_t dyn_off,
                        void* stream);
/* In place: logits -> (softmax - onehot) * (n_valid ? 1/max(*n_valid,1) : 1); ignored rows -> 0
 * (the second pass of _ce_fwd_inplace_kernel, fused_linear_cross_entropy.py:66-77). */
int hilda_flce_dlogits(void* logits, const float* lse, const int64_t* targets, int64_t ignore_index,
                       const int* n_valid, int64_t rows, int64_t V, int64_t vocab_start, int dtype,
                       const int* dyn_rows, int64_t dyn_off, void* stream);
/* dh = dlogits @ W (fused_linear_cross_entropy.py:158); exactly one of dh16 / dh32 non-null. */
int hilda_flce_grad_hidden(const void* dlogits, const void* W, void* dh16, float* dh32, int64_t rows, int64_t H,
                           int64_t V, int dtype, int* status, const int* dyn_rows, int64_t dyn_off, void* stream);
/* dW (+)= dlogits^T @ hidden (fused_linear_cross_entropy.py:161). mode 0: dw32 = .; 1: dw32 += .;
 * 2: dw16 = dw32 + .; 3: dw16 = . */
int hilda_flce_grad_weight(const void* dlogits, const void* hidden, float* dw32, void* dw16, int mode,
                           int64_t rows, int64_t H, int64_t V, int dtype, int* status, const int* dyn_rows,
                           int64_t dyn_off, void* stream);
/* *out = sum(rows) (/ max(*n_valid, 1) when divide != 0); NaN if status is given and *status != 0
 * (the final reduction of fused_linear_cross_entropy.py:165-171, on the device). */
int hilda_flce_sum_loss(const float* rows, int64_t n, const int* n_valid, int divide, const int* status, float* out,
                        void* stream);

/* Device-side compaction of the ignored tokens (no counterpart in the reference). hilda_flce_compact:
 * idx int64 [n] = source row of compacted row j (-1 beyond the count), inv int32 [n] = compacted
 * position of row i (-1 if ignored), t_c int64 [n] = targets in compacted order (ignore_index beyond
 * the count), *n_valid = the count. hilda_gather_valid_rows: dst[j,:] = src[idx[j],:] for the leading
 * *n_valid rows, zero rows up to the next multiple of 256, the rest untouched. hilda_scatter_valid_rows:
 * dst[i,:] = inv[i] >= 0 ? src[inv[i],:] : 0 for all n rows. hilda_scatter_valid_f32: the same for one
 * fp32 value per row. Rows of row_bytes (multiple of 16) bytes. */
int hilda_flce_compact(const int64_t* targets, int64_t n, int64_t ignore_index, int64_t* idx, int* inv, int64_t* t_c,
                       int* n_valid, void* stream);
int hilda_gather_valid_rows(const void* src, const int64_t* idx, const int* n_valid, void* dst, int64_t n,
                            int64_t row_bytes, void* stream);
int hilda_scatter_valid_rows(const void* src, const int* inv, void* dst, int64_t n, int64_t row_bytes, void* stream);
int hilda_scatter_valid_f32(const float* in, const int* inv, float* out, int64_t n, void* stream);

/* Measurement hook (no counterpart in the reference): while enabled, every GEMM launch of the
 * FLCE entry points is bracketed by CUDA events on its stream. collect waits for them and returns
 * per kind (0 logits, 1 d hidden, 2 d W) the summed device milliseconds and the launch count
 * (HOST pointers, 3 entries each). enable != 0 also clears the record. */
void hilda_flce_profile(int enable);
int hilda_flce_profile_collect(float* ms_per_kind, int* launches_per_kind);
/* The i-th bracketed launch since the hook was enabled: kind and device milliseconds (HOST
 * pointers); HILDA_ERR_ARG once i is past the last recorded launch. */
int hilda_flce_profile_entry(int i, int* kind, float* ms);

/* Row moves with an index list whose length the host knows (no counterpart in the reference):
 * dst[i,:] = src[idx[i],:] and dst[idx[i],:] = src[i,:] over rows of row_bytes (multiple of 16)
 * bytes; the scatter zero-fills the n_dst_rows rows of dst first. */
int hilda_gather_rows(const void* src, const int64_t* idx, void* dst, int64_t n_idx, int64_t row_bytes, void* stream);
int hilda_scatter_rows(const void* src, const int64_t* idx, void* dst, int64_t n_idx, int64_t n_dst_rows,
                       int64_t row_bytes, void* stream);

/* The setters from here to hilda_gemm_set_probe act on the CALLING HOST THREAD's later launches only
 * (thread-local state), so threads that drive different GPUs do not disturb each other.
 * GEMM variant used by the FLCE entry points (no counterpart in the reference), per use: bit 0 =
 * logits GEMM, bit 1 = d(hidden) GEMM, bit 2 = d(W) GEMM run on CTA pairs (tcgen05 cta_group::2,
 * 256 x 256 tiles over two SMs); a clear bit = one CTA per 128 x 256 tile. hilda_debug_gemm uses
 * pairs when any bit is set. Initial value: environment HILDA_GEMM_PAIR, else the built-in default. */
void hilda_gemm_set_pair(int mask);
int hilda_gemm_get_pair(void);
/* The FLCE GEMMs launch on at most `sms` SMs (0 = all) until set back; used to leave a few SMs to a
 * collective that runs on another stream beside a GEMM. No counterpart in the reference. */
void hilda_gemm_set_sm_limit(int sms);
/* Attempts every bounded mbarrier wait of the GEMM kernels makes before it gives up, writes a code
 * to the status word and lets the CTA return (0 = the default, 2^22). No counterpart in the reference. */
void hilda_gemm_set_wait_cap(unsigned attempts);
/* Tile walk order hilda_debug_gemm uses (1 = M first, 0 = N first); no counterpart in the reference. */
void hilda_debug_gemm_set_order(int m_fast);
/* Cycle counters of the GEMM kernels' role loops, written by every launch while set: device
 * buffer of [SM count][8] int64 {producer wait-for-slot, producer total, issuer wait-for-data,
 * issuer wait-for-accumulator, issuer total, epilogue wait-for-accumulator, epilogue busy, 0};
 * NULL switches it off (the default). dry = 1 is for measurement only (results are garbage): the
 * producer marks its slots full without loading, taking the memory system out of the loop. dry = 2
 * exercises the failure path: the producer neither loads nor signals, every bounded wait runs out,
 * the status word is set and the kernel returns with nothing in flight. */
void hilda_gemm_set_probe(void* buf, int dry);

/* Validation hook: plain C = A x B through the tcgen05 kernel with either operand K-major
 * ([M,K] / [N,K]) or MN-major (stored [K,M] / [K,N]). No counterpart in the reference. */
int hilda_debug_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, void* c16, float* c32, int64_t ldc,
                     int M, int N, int K, int a_mn, int b_mn, int dtype, int mn_lbo, int mn_sbo, int* status,
                     void* stream);

/* ---- KL divergence, JSD, fused linear + JSD ------------------------------------------------ */
/* Replaces kl_div_forward (kernels/kl_div.py:114-137): y_pred log-probs, y_true probs (log-probs
 * when log_target) [n_rows, n_cols] in dtype; loss_rows [n_rows] fp32 = the per-row sums;
 * reduction 0 none, 1 sum, 2 mean (/ (n_rows * n_cols)), 3 batchmean (/ n_rows) -> loss_out. */
int hilda_kl_div_fwd(const void* y_pred, const void* y_true, float* loss_rows, float* loss_out, int64_t n_rows,
                     int64_t n_cols, int reduction, int log_target, float eps, int dtype, void* stream);
/* Replaces kl_div_backward (kernels/kl_div.py:140-165): dy_pred = -y_true (or -exp(y_true)) *
 * grad_out[0] * the reduction's factor; grad_out is a DEVICE fp32 scalar (the reference reads it on
 * the host); reduction 0 uses scale 1 as the reference does. */
int hilda_kl_div_bwd(const void* y_true, void* dy_pred, const float* grad_out, int64_t n_rows, int64_t n_cols,
                     int reduction, int log_target, int dtype, void* stream);
/* Replaces jsd_forward (kernels/jsd.py:97-135): X student, Y teacher log-probs [n_rows, V]; one
 * pass writes dX (already divided by the number of rows whose label != ignore_index; labels may
 * be null), loss_rows and loss_out = their sum. workspace: 4 bytes, needed with labels. */
int hilda_jsd_fwd(const void* X, const void* Y, void* dX, float* loss_rows, float* loss_out, const int64_t* labels,
                  int64_t ignore_index, void* workspace, int64_t n_rows, int64_t V, float beta, int dtype,
                  void* stream);
/* Row pass of fused_linear_jsd_forward (kernels/fused_linear_jsd.py:168-205: _log_softmax_kernel
 * twice, _jsd_kernel, _softmax_grad_kernel) over one row chunk: from the two heads' logits
 * (hilda_flce_logits_scaled scratch layout) and their row statistics (hilda_flce_row_stats) to the
 * student's dlogits, in place over its logits, and the per-row loss. Divisor: *n_valid (device,
 * clamped to 1) when given, else n_norm. */
int hilda_fljsd_dlogits(void* s_logits, const void* t_logits, const float* rowstat_s, const float* rowstat_t,
                        const int64_t* labels, int64_t ignore_index, const int* n_valid, int64_t n_norm,
                        float* loss_rows, int64_t rows, int64_t V, float beta, float inv_temperature, int dtype,
                        void* stream);

/* ---- AttnRes ------------------------------------------------------------------------------ */
/* Replaces attn_res_forward (kernels/attn_res.py:213-260): V [n_blocks, n_tokens, D] in dtype,
 * w_query / w_norm [D] in their own dtypes, n_blocks <= 32; out [n_tokens, D] = sum_i alpha_i v_i
 * with alpha = softmax_i <w_query, RMSNorm(v_i) * w_norm>; alpha and rstd [n_blocks, n_tokens]
 * fp32 are saved for the backward. Every block row is read once. */
int hilda_attn_res_fwd(const void* V, const void* w_query, const void* w_norm, void* out, float* alpha, float* rstd,
                       int64_t n_blocks, int64_t n_tokens, int64_t D, float eps, int dtype, int wq_dtype,
                       int wn_dtype, void* stream);
/* Replaces attn_res_backward (kernels/attn_res.py:263-293): dV in dtype, dw_query / dw_norm in the
 * weights' dtypes (summed in fp32 in a fixed order; the reference uses float atomics). */
int64_t hilda_attn_res_bwd_workspace_bytes(int64_t n_tokens, int64_t D);
int hilda_attn_res_bwd(const void* d_out, const void* V, const void* w_query, const void* w_norm, const float* alpha,
                       const float* rstd, void* dV, void* dw_query, void* dw_norm, void* workspace,
                       int64_t n_blocks, int64_t n_tokens, int64_t D, int dtype, int wq_dtype, int wn_dtype,
                       void* stream);

/* Kernels of hilda_attn_res_fwd / _bwd: 0 = the reductions over D on the CUDA cores, 1 (default) =
 * on the tensor cores (mma.sync; 16-bit data, n_blocks <= 8, D % 64 == 0, and for the forward both
 * weights in the data's type; anything else runs the kernels of 0). Environment: HILDA_AR_PATH.
 * Returns the previous choice. */
int hilda_attn_res_set_path(int path);

/* ---- Paged FP8 decode attention ----------------------------------------------------------- */
/* Replaces hilda_paged_attention_fp8_decode (kernels/paged_attention_fp8.py:141-188): one query
 * token per sequence. q [batch, n_heads, 128] bf16 (element strides q_sb, q_sh), k_cache / v_cache
 * [blocks, block_size, n_kv_heads, 128] fp8 e4m3 (byte strides per block, token, kv head; multiples
 * of 16), block_tables int32 [batch, max_blocks] (row stride bt_sb), context_lens int32 [batch],
 * out [batch, n_heads, 128] bf16. n_heads % n_kv_heads == 0 (GQA); head_dim must be 128 as in the
 * reference (:134). workspace: hilda_paged_attention_fp8_workspace_bytes(...) bytes (partial
 * results of the context splits). */
int64_t hilda_paged_attention_fp8_workspace_bytes(int64_t batch, int64_t n_heads, int64_t n_kv_heads,
                                                  int64_t max_blocks, int64_t block_size);
int hilda_paged_attention_fp8_decode(const void* q, int64_t q_sb, int64_t q_sh, const void* k_cache, int64_t k_sblk,
                                     int64_t k_stok, int64_t k_sh, const void* v_cache, int64_t v_sblk,
                                     int64_t v_stok, int64_t v_sh, void* out, int64_t o_sb, int64_t o_sh,
                                     const int32_t* block_tables, int64_t bt_sb, const int32_t* context_lens,
                                     void* workspace, float scale, int64_t batch, int64_t n_heads,
                                     int64_t n_kv_heads, int64_t head_dim, int64_t block_size, int64_t max_blocks,
                                     void* stream);


/* ---- GRPO --------------------------------------------------------------------------------- */
int64_t hilda_grpo_workspace_bytes(int64_t B);
/* Replaces grpo_loss_forward + grpo_loss_backward (kernels/grpo_loss.py:241-297, :300-330) in one
 * pass. logits [B, L+1, V]; ids [B, L] int64; mask [B, L] fp32 or null (0 = token skipped; otherwise its weight in the
 * reductions, the reference's completion_mask.float(), grpo_loss.py:264); advantages [B] fp32;
 * old_logp/ref_logp [B, L] fp32 or null. Per-token fp32 outputs loss/kl/clipped/lse [B, L];
 * scalars_out[4] = {loss, kl_mean, clip_ratio, sum(mask)}; B_total > 0 normalises loss and gradient by
 * B_total sequences instead of B (sequences sharded over ranks). grad (nullable): d loss / d logits for a unit
 * upstream gradient, [B, L+1, V] in dtype, last position and masked tokens zero. */
int hilda_grpo_loss_fwd(const void* logits, const int64_t* ids, const float* advantages, const float* old_logp,
                        const float* ref_logp, const float* mask, void* grad, float* loss, float* kl,
                        float* clipped, float* lse, float* scalars_out, void* workspace, int64_t B, int64_t L,
                        int64_t V, int64_t B_total, float temperature, float beta, float eps_low, float eps_high,
                        int dtype, void* stream);

/* Replaces fused_selective_log_softmax (kernels/grpo_loss.py:65-80). */
int hilda_selective_log_softmax(const void* logits, const int64_t* ids, const float* mask, float* logp,
                                int64_t B, int64_t L, int64_t V, float temperature, int dtype, void* stream);

/* Tuning hook for the row engine behind CrossEntropy/GRPO: force (register vectors per thread, CTAs
 * per cluster, shared-memory vectors per thread); (0, 0, 0) restores the automatic plan. Acts on the
 * calling host thread only. No counterpart in the reference. */
void hilda_row_engine_force(int nv, int cluster, int ns);

/* Host-only queries (no GPU needed, no counterpart in the reference): the plan the row engine takes
 * for rows of V elements of `dtype` on 16-byte aligned tensors, out = {threads, register vectors per
 * thread, CTAs per cluster, shared-memory vectors per thread}; returns 1, or 0 when the scalar kernel
 * serves the shape. hilda_row_engine_has_kernel: 1 if the kernel is instantiated for that plan. */
int hilda_row_engine_plan(int64_t V, int dtype, int* out);
int hilda_row_engine_has_kernel(int threads, int nv, int cluster, int ns);

#ifdef __cplusplus
}
#endif
#endif /* HILDA_B200_H */
