/* C ABI of libcustom_cuda_b200.so - B200 (sm_100a) kernels for the Llama-block ops.
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes,
 * returns a cudaError_t as int32_t (0 = success), launches asynchronously on
 * the given stream (a cudaStream_t passed as void*), and - unless stated
 * otherwise - never allocates, frees, copies or synchronises.  All buffers
 * are owned by the caller, row-major and contiguous.  `dtype` is one of the
 * CCK_* tags below; empty problems return success without launching.
 *
 * The first seven functions are binary-compatible replacements for the
 * launchers the reference project (BhargavKumarNath/custom_cuda_kernals)
 * binds from Rust; each comment cites the declaration it replaces.  The rest
 * are additions that follow the same conventions.
 */
#ifndef CUSTOM_CUDA_B200_H_
#define CUSTOM_CUDA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype tags; values fixed by csrc/includes/common.cuh:28-34 and src/kernels/dtype.rs:6-12 */
enum {
    CCK_F32 = 0,
    CCK_F16 = 1,
    CCK_BF16 = 2,
    CCK_F8E4M3 = 3,
    CCK_F8E5M2 = 4
};

/* residual_out = x + residual;  y = residual_out * rsqrt(mean(residual_out^2) + eps) * weight.
 * x, residual, y, residual_out: [rows, cols]; weight: [cols]; one dtype (f32/f16/bf16).
 * Replaces csrc/includes/rmsnorm_residual.h:17-27. */
int32_t launch_rmsnorm_residual_fwd(const void* x, const void* residual, const void* weight, void* y,
                                    void* residual_out, int64_t rows, int64_t cols, float eps,
                                    int32_t dtype, void* stream);

/* y = silu(gate) * up over n elements.  Replaces csrc/includes/swiglu.h:16-22. */
int32_t launch_swiglu_fwd(const void* gate, const void* up, void* y, int64_t n, int32_t dtype, void* stream);

/* Half-split rotary embedding of q [batch, seq_len, n_q_heads, head_dim] and
 * k [batch, seq_len, n_kv_heads, head_dim]; cos_table/sin_table [seq_len, head_dim/2] float32.
 * head_dim must be even.  Replaces csrc/includes/rope.h:23-36. */
int32_t launch_rope_fwd(const void* q, const void* k, const void* cos_table, const void* sin_table,
                        void* q_out, void* k_out, int64_t batch, int64_t seq_len, int64_t n_q_heads,
                        int64_t n_kv_heads, int64_t head_dim, int32_t dtype, void* stream);

/* FP8 quantisation with one scale per 128x128 tile: scale = max(amax/FP8_MAX, 1e-12),
 * x_fp8 = fp8(x / scale).  x [m, n]; x_fp8 [m, n] bytes; scale [ceil(m/128), ceil(n/128)].
 * fp8_format is CCK_F8E4M3 or CCK_F8E5M2.  Replaces csrc/includes/fp8_quant.h:41-49. */
int32_t launch_fp8_quant_block_fwd(const void* x, uint8_t* x_fp8, float* scale, int64_t m, int64_t n,
                                   int32_t dtype, int32_t fp8_format, void* stream);

/* FP8 quantisation with one scale for the whole matrix (two kernels on the stream).
 * scale [1]; amax_scratch [1] int32, zeroed by the caller before every call.
 * Replaces csrc/includes/fp8_quant.h:51-60. */
int32_t launch_fp8_quant_tensor_fwd(const void* x, uint8_t* x_fp8, float* scale, int32_t* amax_scratch,
                                    int64_t m, int64_t n, int32_t dtype, int32_t fp8_format, void* stream);

/* y = x @ weight^T + bias.  x [m, k]; weight [n, k]; bias [n] or NULL; y [m, n]; one dtype.
 * Replaces csrc/includes/matmul_add_bias.h:20-29. */
int32_t launch_matmul_add_bias_fwd(const void* x, const void* weight, const void* bias, void* y,
                                   int64_t m, int64_t k, int64_t n, int32_t dtype, void* stream);

/* Online-softmax update with one materialised chunk of logits [n, chunk_v] covering
 * vocabulary columns [v_start, v_start + chunk_v).  running_max / running_sum / target_logit:
 * [n] float32, initialised by the caller to -inf / 0 / 0.  targets [n] int64.
 * Replaces csrc/includes/linear_cross_entropy.h:31-41. */
int32_t launch_linear_ce_chunk_update(const void* logits_chunk, const int64_t* targets, int64_t v_start,
                                      int64_t n, int64_t chunk_v, float* running_max, float* running_sum,
                                      float* target_logit, int32_t dtype, void* stream);

/* ---- additions (no counterpart in the reference) ------------------------------------------ */

/* FP8 quantisation with one scale per row (per token).  scale [m] (viewed as [m, 1]). */
int32_t launch_fp8_quant_token_fwd(const void* x, uint8_t* x_fp8, float* scale, int64_t m, int64_t n,
                                   int32_t dtype, int32_t fp8_format, void* stream);

/* y = (a_codes * a_scale[row]) @ (w_codes * w_scale[col])^T + bias with e4m3 operands.
 * a_codes [m, k], w_codes [n, k] e4m3 bytes; a_scale [m], w_scale [n] float32; bias [n] in
 * out_dtype or NULL; y [m, n] in out_dtype (CCK_BF16 or CCK_F16, else cudaErrorInvalidValue).
 * Every shape runs, like launch_matmul_add_bias_fwd (the reference's launcher falls back for
 * every shape, csrc/kernels/matmul_add_bias.cu:170-180): k % 16 == 0 with 16-byte aligned
 * operands goes to the tensor cores (tcgen05 kind::f8f6f4), anything else to a CUDA-core kernel. */
int32_t launch_matmul_add_bias_fp8_fwd(const uint8_t* a_codes, const float* a_scale, const uint8_t* w_codes,
                                       const float* w_scale, const void* bias, void* y, int64_t m, int64_t k,
                                       int64_t n, int32_t out_dtype, void* stream);

/* Fused linear + softmax statistics, logits never materialised.  hidden [n, h]; weight
 * [v_count, h] = rows v_start .. v_start+v_count-1 of the LM head; targets [n] int64 global ids.
 * row_stats [3][n] float32 receives per row: max logit, sum exp(logit - max), target logit
 * (0 when the target is outside this slice).  workspace: at least cck_lce_workspace_bytes(n,
 * v_count) bytes of device memory, contents irrelevant.  dtype CCK_BF16 or CCK_F16, h % 8 == 0,
 * 16-byte aligned operands; otherwise cudaErrorInvalidValue. */
int32_t launch_linear_cross_entropy_fwd(const void* hidden, const void* weight, const int64_t* targets,
                                        int64_t v_start, int64_t n, int64_t h, int64_t v_count,
                                        float* row_stats, void* workspace, int64_t workspace_bytes,
                                        int32_t dtype, void* stream);
int64_t cck_lce_workspace_bytes(int64_t n, int64_t v_count);
int64_t cck_lce_num_splits(int64_t n, int64_t v_count);

/* No counterpart in the reference.  launch_linear_cross_entropy_fwd for callers that cannot
 * provide (or allocate) a workspace - a server whose memory pool owns all device memory, a loop
 * that must not call cudaMalloc: the workspace is a fixed 6 MiB device array inside the library,
 * held by every GPU that loads it.  No allocation or free is made.  Returns
 * cudaErrorInvalidValue, launching nothing, when cck_lce_workspace_bytes(n, v_count) exceeds
 * cck_lce_noalloc_max_workspace_bytes().  The first call on a device looks up the array's
 * address and should be made outside stream capture (host threads may make it concurrently: each
 * caches the same address).  Calls share the array: calls that overlap on the GPU race and must
 * be serialised by the caller. */
int32_t launch_linear_cross_entropy_fwd_noalloc(const void* hidden, const void* weight, const int64_t* targets,
                                                int64_t v_start, int64_t n, int64_t h, int64_t v_count,
                                                float* row_stats, int32_t dtype, void* stream);
int64_t cck_lce_noalloc_max_workspace_bytes(void);

/* Merge row_stats of n_shards vocabulary slices (stats [n_shards][3][n]) into per-row losses:
 * loss_rows [n] (0 where targets == ignore_index; may be NULL) and reduce_out [2] =
 * { sum of losses, number of rows whose target is not ignore_index }. */
int32_t launch_lce_finalize(const float* stats, const int64_t* targets, int64_t n, int64_t n_shards,
                            int64_t ignore_index, float* loss_rows, float* reduce_out, void* stream);

/* y = x * rsqrt(mean(x^2) + eps) * weight - the norm of launch_rmsnorm_residual_fwd alone, for
 * callers whose residual add already happened in the producing GEMM's epilogue.  x, y [rows, cols];
 * weight [cols]; one dtype.  Equals launch_rmsnorm_residual_fwd with a zero residual. */
int32_t launch_rmsnorm_fwd(const void* x, const void* weight, void* y, int64_t rows, int64_t cols, float eps,
                           int32_t dtype, void* stream);

/* launch_rope_fwd for inputs whose tokens are not packed: consecutive tokens of q (k) are
 * q_token_stride (k_token_stride) elements apart - e.g. q and k are column ranges of one fused
 * QKV projection output [tokens, (Hq + 2 Hkv) * D].  Heads of one token are contiguous; q_out and
 * k_out are contiguous [batch, seq_len, heads, head_dim]. */
int32_t launch_rope_strided_fwd(const void* q, const void* k, const void* cos_table, const void* sin_table,
                                void* q_out, void* k_out, int64_t batch, int64_t seq_len, int64_t n_q_heads,
                                int64_t n_kv_heads, int64_t head_dim, int64_t q_token_stride,
                                int64_t k_token_stride, int32_t dtype, void* stream);

/* Fused gate/up projection + SwiGLU: y[m, f] = silu(x @ Wg^T) * (x @ Wu^T).  w_gate_up is
 * [2f, k]: for every block j of 128 output features, rows [256j, 256j+128) hold rows
 * [128j, 128j+128) of Wg and rows [256j+128, 256j+256) the same rows of Wu.  Rounds where the
 * unfused chain rounds (launch_matmul_add_bias_fwd twice, then launch_swiglu_fwd), so the result
 * is identical.  dtype CCK_BF16 or CCK_F16; f % 128 == 0, k % 8 == 0, 16-byte aligned operands;
 * otherwise cudaErrorInvalidValue. */
int32_t launch_matmul_swiglu_fwd(const void* x, const void* w_gate_up, void* y, int64_t m, int64_t k,
                                 int64_t f, int32_t dtype, void* stream);

/* Fused q/k/v projection + rotary embedding: y[m, n] = x @ weight^T + bias with RoPE (half-split
 * convention, heads of 128 columns: column j of a head rotates with column j + 64) applied to the
 * columns below rope_cols - the q and k heads - and the rest (v) stored as projected.  Row r is
 * position r % seq_len; cos_table / sin_table are [seq_len, 64] float32.  The projection is rounded
 * to the storage type before the rotation, so the result is identical to launch_matmul_add_bias_fwd
 * followed by launch_rope_strided_fwd on the q and k column ranges (the steps of
 * examples/llama_block.py:147-156 for a concatenated q/k/v weight).  dtype CCK_BF16 or CCK_F16;
 * n % 128 == 0, rope_cols % 128 == 0, rope_cols <= n, k % 8 == 0, 16-byte aligned operands and
 * tables; otherwise cudaErrorInvalidValue.  No reference counterpart. */
int32_t launch_matmul_add_bias_rope_fwd(const void* x, const void* weight, const void* bias,
                                        const float* cos_table, const float* sin_table, void* y, int64_t m,
                                        int64_t k, int64_t n, int64_t rope_cols, int64_t seq_len,
                                        int32_t dtype, void* stream);

/* y = x @ weight^T + bias + residual (residual [m, n], bias [n] or NULL), identical to
 * launch_matmul_add_bias_fwd followed by an elementwise add in the storage type.  dtype CCK_BF16
 * or CCK_F16; k % 8 == 0, 16-byte aligned x and weight; otherwise cudaErrorInvalidValue. */
int32_t launch_matmul_add_bias_residual_fwd(const void* x, const void* weight, const void* bias,
                                            const void* residual, void* y, int64_t m, int64_t k, int64_t n,
                                            int32_t dtype, void* stream);

/* Backward helper of the linear cross entropy (the reference is forward-only): d(loss)/d(logits)
 * for rows [0, n) over the whole vocabulary, dlogits[i, j] = (exp(logit_ij - lse[i]) - [j ==
 * targets[i]]) * grad_scale, 0 for rows whose target is ignore_index, written as [n, v] in the
 * storage type.  The logits are recomputed by the tensor-core mainloop and never stored.
 * lse[i] = max + log(sum-exp) of row i from launch_linear_cross_entropy_fwd's row_stats.
 * dtype CCK_BF16 or CCK_F16, h % 8 == 0, aligned operands; otherwise cudaErrorInvalidValue. */
int32_t launch_lce_dlogits_fwd(const void* hidden, const void* weight, const int64_t* targets, const float* lse,
                               int64_t n, int64_t h, int64_t v, int64_t ignore_index, float grad_scale,
                               void* dlogits, int32_t dtype, void* stream);

/* launch_linear_cross_entropy_fwd that also leaves the fp32 logits in logits[n, v_count]
 * (v_count % 4 == 0, 16-byte aligned) for launch_lce_dlogits_from_logits - the gradient path
 * then reads them once instead of running the contraction a second time.  No reference
 * counterpart. */
int32_t launch_linear_cross_entropy_fwd_store(const void* hidden, const void* weight, const int64_t* targets,
                                              int64_t v_start, int64_t n, int64_t h, int64_t v_count,
                                              float* row_stats, void* workspace, int64_t workspace_bytes,
                                              float* logits, int32_t dtype, void* stream);

/* d(loss)/d(logits) from stored fp32 logits[n, v] (formula of launch_lce_dlogits_fwd), written
 * both as dlogits[n, v] and transposed as dlogits_t[v, ld_t] (ld_t >= n, a multiple of 4; columns
 * n..ld_t are left untouched) in the storage type `dtype` (CCK_BF16 / CCK_F16).  targets index
 * the columns of logits; a value outside [0, v) selects none.  v % 4 == 0; logits 16-byte,
 * dlogits and dlogits_t 8-byte aligned.  No reference counterpart. */
int32_t launch_lce_dlogits_from_logits(const float* logits, const int64_t* targets, const float* lse, int64_t n,
                                       int64_t v, int64_t ignore_index, float grad_scale, void* dlogits,
                                       void* dlogits_t, int64_t ld_t, int32_t dtype, void* stream);

/* ---- Mixture-of-experts neighbours of the block (reference csrc/includes/moe_router.h:20-29,
 * csrc/includes/token_permute.h:17-41): same signatures and semantics. */

/* probs = softmax(logits[t, :]) in fp32; topk_weights[t, :k] / topk_indices[t, :k] = the k largest
 * probabilities (descending; ties to the lower expert id) and their expert ids; with renormalize
 * the k weights are divided by their sum.  logits [num_tokens, num_experts] in `dtype`,
 * num_experts <= 256 and 0 < k <= num_experts, else cudaErrorInvalidValue. */
int32_t launch_moe_router_fwd(const void* logits, float* topk_weights, int64_t* topk_indices, int64_t num_tokens,
                              int64_t num_experts, int64_t k, int32_t dtype, int32_t renormalize, void* stream);

/* dst[i, :] = src[indices[i], :] for i < n_dst_rows; indices must lie inside src. */
int32_t launch_token_gather_fwd(const void* src, const int64_t* indices, void* dst, int64_t n_dst_rows,
                                int64_t hidden_dim, int32_t dtype, void* stream);

/* combined[t, :] = sum_j weights[t, j] * expert_output[unpermute_index[t, j], :], accumulated in
 * fp32, one rounding.  unpermute_index, weights: [n_tokens, k]; weights float32. */
int32_t launch_token_combine_fwd(const void* expert_output, const int64_t* unpermute_index, const float* weights,
                                 void* combined, int64_t n_tokens, int64_t k, int64_t hidden_dim, int32_t dtype,
                                 void* stream);

/* Expert-parallel forms of the two row movers (no reference counterpart): the destination /
 * source of a row is (rank, row) - an entry of a device array of `world` buffer base addresses
 * (this GPU's own receive buffer and its peers' buffers mapped into this process) and a row
 * index.  Push / pull only: nothing waits on another GPU inside the kernels; separate the
 * phases with stream-ordered barriers.  hidden_dim * element size must be a multiple of 16,
 * every buffer 16-byte aligned.  A route outside [0, world) x [0, capacity_rows) (or a source
 * row outside [0, n_src_rows)) is skipped and sets bit 2 of cck_take_device_status(). */
int32_t launch_token_dispatch_fwd(const void* src, const int64_t* src_row, const int64_t* dst_rank,
                                  const int64_t* dst_row, const int64_t* dst_bases, int64_t world,
                                  int64_t capacity_rows, int64_t n_src_rows, int64_t n, int64_t hidden_dim,
                                  int32_t dtype, void* stream);
/* The routes of one expert-parallel call in one launch: topk = this rank's n = tokens x k flattened
 * expert ids, counts = [world, experts] all-gathered per-expert counts (int64).  Writes, all int64:
 * src_row / dst_rank / dst_row [n] in expert-sorted slot order (a stable sort: pairs of one expert keep
 * their order) - the arguments of launch_token_dispatch_fwd; pull_rank / pull_row [n] in (token, choice)
 * order - the arguments of launch_token_combine_remote_fwd; meta[0] = rows this rank receives, meta[1] =
 * the most rows any rank receives.  A rank's receive buffer holds blocks in source-rank order, each
 * sorted by expert.  experts <= 256, world <= 32, experts % world == 0, else cudaErrorInvalidValue. */
int32_t launch_ep_plan(const int64_t* topk, const int64_t* counts, int64_t n, int64_t k, int64_t world,
                       int64_t experts, int64_t rank, int64_t* src_row, int64_t* dst_rank, int64_t* dst_row,
                       int64_t* pull_rank, int64_t* pull_row, int64_t* meta, void* stream);
int32_t launch_token_combine_remote_fwd(const int64_t* src_bases, int64_t world, int64_t capacity_rows,
                                        const int64_t* src_rank, const int64_t* src_row, const float* weights,
                                        void* combined, int64_t n_tokens, int64_t k, int64_t hidden_dim, int32_t dtype,
                                        void* stream);

/* Gradients of launch_swiglu_fwd for an upstream gradient dy: dgate = dy * up * silu'(gate),
 * dup = dy * silu(gate), flat over n elements, fp32 arithmetic, one rounding.  No reference
 * counterpart (the reference is forward-only). */
int32_t launch_swiglu_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup, int64_t n,
                          int32_t dtype, void* stream);

/* Gradients of launch_rmsnorm_residual_fwd.  Inputs: dy, the saved residual_out, weight, and
 * d_residual_out - the gradient arriving through the second output, or NULL.  Outputs: dx
 * (the gradient of x and, being equal, of residual) and dweight [cols] in the storage type.
 * workspace: cck_rmsnorm_bwd_workspace_bytes(rows, cols) bytes of device memory.  cols must be a
 * multiple of the 16-byte vector width and at most 8192 (16-bit) / 4096 (fp32), every pointer
 * 16-byte aligned; otherwise cudaErrorInvalidValue.  No reference counterpart. */
int64_t cck_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t cols);
int32_t launch_rmsnorm_residual_bwd(const void* dy, const void* d_residual_out, const void* residual_out,
                                    const void* weight, void* dx, void* dweight, void* workspace,
                                    int64_t workspace_bytes, int64_t rows, int64_t cols, float eps, int32_t dtype,
                                    void* stream);

/* out[c, r] = in[r, c] for a contiguous [rows, cols] matrix of 2-byte elements (float16 or
 * bfloat16); out is [cols, ld_out], ld_out >= rows, and out[:, rows..ld_out) is zero-filled.
 * cols % 4 == 0, ld_out % 4 == 0, 8-byte aligned pointers.  Makes the row-contiguous operands
 * (hidden^T, W^T) of the gradient GEMMs.  No reference counterpart. */
int32_t launch_transpose_2byte(const void* in, int64_t rows, int64_t cols, void* out, int64_t ld_out, void* stream);

/* y[m, n] (float32) += x[m, k] @ weight[n, k]^T with 16-bit operands: a GEMM that accumulates
 * into its output across calls (a weight gradient summed over row blocks).  k % 8 == 0,
 * 16-byte aligned x, weight and y; otherwise cudaErrorInvalidValue. */
int32_t launch_matmul_accumulate_f32_fwd(const void* x, const void* weight, float* y, int64_t m, int64_t k,
                                         int64_t n, int32_t dtype, void* stream);

/* y = x @ weight^T + bias (+ residual when not NULL): bit for bit what launch_matmul_add_bias_fwd
 * (or launch_matmul_add_bias_residual_fwd) stores, and in the same epilogue the statistics the op
 * AFTER the GEMM needs, per row and per 256-column output tile, taken from the stored (rounded)
 * values: row_sumsq[t][row] = sum of squares, row_amax[t][row] = largest magnitude, each
 * [cck_gemm_stat_tiles(n), m] float32, either may be NULL.  A row's tiles are computed by
 * different CTAs, so the row-wide reduction is the consumer's (n_tiles values per row):
 * launch_rmsnorm_from_stats_fwd and launch_fp8_quant_token_from_amax_fwd.  float16/bfloat16,
 * k % 8 == 0, 16-byte aligned x and weight; otherwise cudaErrorInvalidValue.  These are the steps
 * either side of the projections in the reference's decoder block (examples/llama_block.py:163-172:
 * o_proj -> norm, down_proj -> next norm); the reference has no fused form of them. */
int64_t cck_gemm_stat_tiles(int64_t n);
int32_t launch_matmul_add_bias_stats_fwd(const void* x, const void* weight, const void* bias, const void* residual,
                                         void* y, float* row_sumsq, float* row_amax, int64_t m, int64_t k,
                                         int64_t n, int32_t dtype, void* stream);

/* y = x * rsqrt(sum_t row_sumsq[t][row] / cols + eps) * weight: launch_rmsnorm_fwd for rows whose sums
 * of squares the producing GEMM left as n_tiles partials per row.  Same rounding chain; the
 * statistic differs from launch_rmsnorm_fwd's only in the order of its fp32 additions.
 * float16/bfloat16, cols a multiple of 8 and at most 65536, 16-byte aligned pointers; otherwise
 * cudaErrorInvalidValue.  No reference counterpart. */
int32_t launch_rmsnorm_from_stats_fwd(const void* x, const float* row_sumsq, int64_t n_tiles, const void* weight,
                                      void* y, int64_t rows, int64_t cols, float eps, int32_t dtype, void* stream);

/* launch_fp8_quant_token_fwd for rows whose largest magnitudes the producing GEMM left as n_tiles
 * partial maxima per row (row_amax [n_tiles, m]); codes and scales are bit for bit the same.
 * float16/bfloat16, n a multiple of 8 and at most 65536, x 16-byte and x_fp8 8-byte aligned;
 * otherwise cudaErrorInvalidValue.  No reference counterpart. */
int32_t launch_fp8_quant_token_from_amax_fwd(const void* x, const float* row_amax, int64_t n_tiles, uint8_t* x_fp8,
                                             float* scale, int64_t m, int64_t n, int32_t dtype, int32_t fp8_format,
                                             void* stream);

/* x_fp8, scale = launch_fp8_quant_token_fwd(launch_rmsnorm_fwd(x, weight, eps)), bit for bit, in ONE
 * pass over x: the normalised row stays in registers between the norm and the quantiser (3 bytes of
 * HBM traffic per element instead of 7).  row_sumsq, when not NULL, holds n_tiles partial sums of
 * squares per row ([n_tiles, rows], from launch_matmul_add_bias_stats_fwd) and replaces the row
 * reduction.  y, when not NULL, also receives the normalised rows.  float16/bfloat16, cols a multiple
 * of 8 and at most 65536, 16-byte aligned x, weight, y, 8-byte aligned x_fp8; otherwise
 * cudaErrorInvalidValue.  The norm -> projection step of the reference's block
 * (examples/llama_block.py:161-163,168-170) for FP8 projections; no reference counterpart. */
int32_t launch_rmsnorm_fp8_quant_token_fwd(const void* x, const void* weight, const float* row_sumsq, int64_t n_tiles,
                                           void* y, uint8_t* x_fp8, float* scale, int64_t rows, int64_t cols,
                                           float eps, int32_t dtype, int32_t fp8_format, void* stream);

/* launch_matmul_add_bias_rope_fwd with e4m3 operands: y = rope(a_scale[row] * w_scale[col] * (codes @
 * codes^T) + bias) on the columns below rope_cols, as projected on the rest; identical to
 * launch_matmul_add_bias_fp8_fwd followed by launch_rope_strided_fwd on the q and k column ranges.
 * out_dtype CCK_BF16 or CCK_F16; n % 128 == 0, rope_cols % 128 == 0, k % 16 == 0, 16-byte aligned
 * codes and tables; otherwise cudaErrorInvalidValue.  No reference counterpart. */
int32_t launch_matmul_add_bias_rope_fp8_fwd(const uint8_t* a_codes, const float* a_scale, const uint8_t* w_codes,
                                            const float* w_scale, const void* bias, const float* cos_table,
                                            const float* sin_table, void* y, int64_t m, int64_t k, int64_t n,
                                            int64_t rope_cols, int64_t seq_len, int32_t out_dtype, void* stream);

/* FP8 forms of launch_matmul_swiglu_fwd and launch_matmul_add_bias_residual_fwd: e4m3 codes with one
 * float32 scale per row of each operand (as launch_fp8_quant_token_fwd produces; the weight's scales
 * are per output channel).  Results equal, bit for bit, launch_matmul_add_bias_fp8_fwd followed by
 * launch_swiglu_fwd / the residual add.  w_gate_up [2 f, k] and w_scale [2 f] are in the interleaved
 * row order of launch_matmul_swiglu_fwd; row_amax [f / 128, m] (or NULL) receives each row's largest
 * stored magnitude per 128 output columns, for launch_fp8_quant_token_from_amax_fwd.  k % 16 == 0,
 * f % 128 == 0, 16-byte aligned codes; out_dtype CCK_BF16 or CCK_F16; otherwise
 * cudaErrorInvalidValue.  No reference counterpart. */
int32_t launch_matmul_swiglu_fp8_fwd(const uint8_t* a_codes, const float* a_scale, const uint8_t* w_gate_up,
                                     const float* w_scale, void* y, float* row_amax, int64_t m, int64_t k, int64_t f,
                                     int32_t out_dtype, void* stream);
int32_t launch_matmul_add_bias_residual_fp8_fwd(const uint8_t* a_codes, const float* a_scale, const uint8_t* w_codes,
                                                const float* w_scale, const void* bias, const void* residual, void* y,
                                                int64_t m, int64_t k, int64_t n, int32_t out_dtype, void* stream);

/* y[m, n] = A B^T on the tensor cores with either operand read as stored: A [m, k] (a_is_km = 0) or
 * its transpose [k, m] (a_is_km = 1); B [n, k] (b_is_kn = 0, the reference's weight layout,
 * custom_cuda/kernels/matmul_add_bias.py:16-26) or its transpose [k, n] (b_is_kn = 1).  The
 * gradient GEMMs of a linear layer, dX = dY W and dW = dY^T X, are the transposed forms; no
 * transposed copy of an operand is made (MN-major tcgen05 descriptors).  accumulate_f32 = 0: y in
 * `dtype`, overwritten; 1: y float32, the product is added to it.  float16 / bfloat16; the
 * contiguous dimension of each operand a multiple of 8, pointers 16-byte aligned; otherwise
 * cudaErrorInvalidValue.  No reference counterpart (the reference is forward-only). */
int32_t launch_matmul_general_fwd(const void* a, const void* b, void* y, int64_t m, int64_t k, int64_t n,
                                  int32_t a_is_km, int32_t b_is_kn, int32_t accumulate_f32, int32_t dtype,
                                  void* stream);

/* Number of two-CTA pairs the tensor-core GEMM keeps resident on the current device; 0 means
 * the pair kernel is unavailable (or disabled with CCK_GEMM_SINGLE_CTA=1) and the single-CTA
 * kernel is used. */
int32_t cck_gemm_pair_capacity(void);

/* Reads and clears the error word of the tensor-core kernels on the current device (bit 0: a
 * bounded wait inside a kernel ran out and the kernel gave up).  Synchronises the device. */
int32_t cck_take_device_status(uint32_t* out);

/* Limit, in nanoseconds of the GPU's global timer, of every bounded wait inside this library's
 * kernels on the current device (mbarrier waits of the tensor-core GEMMs and of the TMA-staged
 * FP8 block quantiser).  The library starts with 2 s; values are clamped to [1 us, 10 s].  The
 * previous limit is returned in *previous_ns (may be NULL).  Synchronises the device.  No
 * reference counterpart: the reference's kernels never wait. */
int32_t cck_set_wait_limit_ns(uint64_t limit_ns, uint64_t* previous_ns);

/* Self-test of the give-up path: launches ONE tile of a real GEMM kernel whose A tensor map
 * delivers half the bytes the kernel's "stage full" barrier counts on, so that barrier never
 * completes, no MMA is issued, and the waiting roles run into the wait limit.  Expected outcome:
 * the kernel returns by itself, y is left unwritten, cck_take_device_status() reports bit 0, and
 * the next launch works (tensor memory was freed).  Nothing faults.  Call cck_set_wait_limit_ns
 * with about a millisecond first and restore the limit afterwards.
 *   a, b: [256, 64] bfloat16 each (16-byte aligned), y: [256, 256] bfloat16
 *   variant 0: single-CTA kernel, 1: CTA-pair kernel (cta_group::2), 2: cluster split-K kernel
 * No reference counterpart. */
int32_t launch_wait_limit_selftest(const void* a, const void* b, void* y, int32_t variant, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CUSTOM_CUDA_B200_H_ */
