/*
 * tb200 — C ABI of the sm_100a kernels behind the PCVR inference hot path.
 *
 * Conventions shared by every entry point:
 *   - plain C types only; all data pointers are DEVICE pointers owned by the caller and
 *     kept alive until the stream has passed the call;
 *   - the work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream); no entry point synchronises, allocates device memory or
 *     takes ownership of anything unless its comment says so;
 *   - the return value is 0 on success, a negative TB200_ERR_* code for a rejected
 *     argument (nothing was launched), or a positive cudaError_t from the launch;
 *   - tensors are dense row-major unless strides are passed explicitly.
 *
 * Each declaration names the reference operator it stands behind
 * (paths are relative to the reference project's root).
 */
#ifndef TB200_H_
#define TB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------------------- */
#define TB200_OK 0
#define TB200_ERR_NULL (-1)        /* a required pointer is NULL */
#define TB200_ERR_DTYPE (-2)       /* unknown / unsupported element or index type */
#define TB200_ERR_SHAPE (-3)       /* a size is negative, zero where it must not be, or too large */
#define TB200_ERR_ALIGN (-4)       /* a pointer or stride breaks the kernel's alignment rule */
#define TB200_ERR_UNSUPPORTED (-5) /* valid request that this build has no kernel for */
#define TB200_ERR_DEVICE (-6)      /* current device is not compute capability 10.x */
#define TB200_ERR_DRIVER (-7)      /* a driver entry point (tensor-map encode) is unavailable or failed */
#define TB200_ERR_SCRATCH (-8)     /* the request does not fit the fixed scratch of a no-allocation entry point */
#define TB200_ERR_RANGE (-9)       /* a value does not fit the 32-bit compact host format: use the padded 64-bit copy */

/* ---- element / index type codes ------------------------------------------------------- */
#define TB200_F32 0
#define TB200_F16 1
#define TB200_BF16 2
#define TB200_I32 0
#define TB200_I64 1

/* Human-readable text for a status code returned by this library (never NULL). */
const char* tb200_strerror(int code);

/* Library ABI version; bumped when a signature changes. */
int tb200_abi_version(void);

/* 1 if the CURRENT device can run these kernels (compute capability 10.x), else 0.
 * Mirrors the availability probes the reference dispatchers consult before choosing an
 * accelerated backend (src/taac2026/infrastructure/accelerators/tilelang_runtime.py,
 * triton_runtime.py). */
int tb200_device_ok(void);

/* Number of kernel launches enqueued by this library in this process so far. */
int64_t tb200_launch_count(void);

/* ---- (b) normalisation ------------------------------------------------------------------
 * y[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * gamma          (fp32 accumulation)
 * Replaces the accelerated branches of `rms_norm`
 * (src/taac2026/infrastructure/accelerators/normalization/rms_norm.py:377-401; oracle
 * `_torch_rms_norm` :71-73).  x, y: [rows, cols] contiguous, gamma: [cols], all of
 * `dtype`.  rows may be 0.  Any cols >= 1 is accepted; rows whose byte length is a multiple
 * of 16 with 16-byte aligned bases take the TMA-staged kernel. */
int tb200_rmsnorm_fwd(const void* x, const void* gamma, void* y, int64_t rows, int32_t cols, float eps, int dtype,
                      void* stream);

/* y[r, :] = (x[r, :] - mean) * rsqrt(var + eps) * gamma + beta, two-pass centred variance in fp32.
 * Replaces the accelerated branch of `layer_norm`
 * (src/taac2026/infrastructure/accelerators/normalization/layer_norm.py:261-280; oracle
 * `_torch_layer_norm` :65-66). */
int tb200_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int32_t cols,
                        float eps, int dtype, void* stream);

/* y = rmsnorm(x + in_bias) * gamma, the bias added in fp32 before the statistics.  In OneTrans's block
 * (`tokens = tokens + attention(...)`, then `ffn_norm(tokens)`, experiments/onetrans/model.py:106-107) the
 * output projection's bias reaches the norm this way, so the residual addition can stay inside the
 * projection GEMM and no separate pass adds the bias.  in_bias: [cols] of `dtype`. */
int tb200_rmsnorm_bias_fwd(const void* x, const void* in_bias, const void* gamma, void* y, int64_t rows, int32_t cols,
                           float eps, int dtype, void* stream);

/* y = layernorm(silu(x)) with the SiLU result rounded to `dtype` first: the tail of the tokenizers'
 * `nn.Sequential(nn.Linear, nn.SiLU(), nn.LayerNorm)` projections
 * (src/taac2026/infrastructure/modeling/tokenizers.py:94, :144) without the intermediate tensor. */
int tb200_layernorm_silu_fwd(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int32_t cols,
                             float eps, int dtype, void* stream);

/* tokens = layernorm(silu(x)) + table_a[ids_a] (+ table_b[ids_b]);  normed = rmsnorm(tokens) * rms_gamma
 * in one pass over the matrix: the tail of the sequence tokenizer (`nn.SiLU(), nn.LayerNorm`, time-bucket
 * and position rows, src/taac2026/infrastructure/modeling/tokenizers.py:144, :188-189) followed by the
 * `attn_norm` of the first `OneTransBlock` (experiments/onetrans/model.py:106).  Every intermediate is rounded to
 * `dtype` where the separate operations would have stored it, so `tokens` equals
 * `tb200_layernorm_silu_fwd` + `tb200_add_gathered_rows` bit for bit and `normed` equals `tb200_rmsnorm_fwd` of
 * it.  Needs rows of whole 16-byte pieces and 16-byte aligned bases (TB200_ERR_UNSUPPORTED otherwise); ids are
 * device int64[rows], clamped into their table; table_b may be NULL. */
int tb200_token_tail_fwd(const void* x, const void* ln_gamma, const void* ln_beta, const void* table_a, int64_t rows_a,
                         const int64_t* ids_a, const void* table_b, int64_t rows_b, const int64_t* ids_b,
                         const void* rms_gamma, void* tokens, void* normed, int64_t rows, int32_t cols, float ln_eps,
                         float rms_eps, int dtype, void* stream);

/* `tb200_token_tail_fwd` with the pyramid's row selection of the first block folded in: `normed` still
 * receives every row (the block projects keys and values from all of them), but `tokens` is written in
 * compacted form, tokens[row_dst[r], :] = row r for 0 <= row_dst[r] < rows_out, and rows with any other
 * `row_dst` are not written at all.  That is `tokens = tokens[:, -next_len:, :]` of
 * `OneTransBlock.forward`'s caller (experiments/onetrans/model.py:176-180) applied to the residual stream before it is stored instead of
 * after.  row_dst: device int32[rows] or NULL (then identical to `tb200_token_tail_fwd`); tokens:
 * [rows_out, cols]. */
int tb200_token_tail_select_fwd(const void* x, const void* ln_gamma, const void* ln_beta, const void* table_a,
                                int64_t rows_a, const int64_t* ids_a, const void* table_b, int64_t rows_b,
                                const int64_t* ids_b, const void* rms_gamma, const int32_t* row_dst, int64_t rows_out,
                                void* tokens, void* normed, int64_t rows, int32_t cols, float ln_eps, float rms_eps,
                                int dtype, void* stream);

/* ---- normalisation backward (training side) ----------------------------------------------
 * Gradients of the two norms above, statistics recomputed from x in fp32:
 *   RMSNorm    dx = r (dy g) - x r^3 mean(dy g x),   dgamma = sum_rows dy x r              (r = rsqrt(mean(x^2) + eps))
 *   LayerNorm  dx = rs (dy g - mean(dy g) - xh mean(dy g xh)),  dgamma = sum_rows dy xh,  dbeta = sum_rows dy
 * Replaces the backward kernels of the reference's accelerated norms
 * (src/taac2026/infrastructure/accelerators/normalization/kernels/triton.py:83-116, :277-320: dX per row, partial
 * dW / dB per block, then a reduction).  x, dy, dx: [rows, cols]; gamma, dgamma, dbeta: [cols]; all of `dtype`.
 * cols must be whole 16-byte pieces and at most 128 of them (1024 columns of a 16-bit type, 512 of fp32);
 * TB200_ERR_UNSUPPORTED otherwise.  workspace: device floats, tb200_norm_bwd_workspace_bytes(cols, layer_norm) bytes,
 * holds the per-CTA partial sums between the two kernels of a call (no other state).  Sums run in a fixed order:
 * the result does not depend on scheduling. */
int64_t tb200_norm_bwd_workspace_bytes(int32_t cols, int32_t layer_norm);
int tb200_rmsnorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, void* dgamma, float* workspace,
                      int64_t rows, int32_t cols, float eps, int dtype, void* stream);
int tb200_layernorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, void* dgamma, void* dbeta,
                        float* workspace, int64_t rows, int32_t cols, float eps, int dtype, void* stream);

/* The whole sequence tokenizer in one kernel: row gather -> projection -> SiLU -> LayerNorm -> time / position rows
 * -> first RMSNorm,
 *     x[r, :]      = concat_f tables[f][clamp(ids[f, r]), :]                     (K = n_feat * emb columns)
 *     tokens[r, :] = layernorm(silu(x[r, :] @ w^T + bias)) + table_a[ids_a[r]] (+ table_b[ids_b[r]])
 *     normed[r, :] = rmsnorm(tokens[r, :]) * rms_gamma
 * i.e. `SequenceTokenizer.forward` (src/taac2026/infrastructure/modeling/tokenizers.py:156-190: `nn.Embedding`
 * lookups, `torch.cat`, `nn.Linear -> nn.SiLU -> nn.LayerNorm`, the time-bucket rows), the sinusoidal position rows and
 * the `attn_norm` of the first `OneTransBlock` (experiments/onetrans/model.py:106) without the gathered [rows, K]
 * matrix and the projected [rows, n_cols] matrix ever being written: tb200_gather_rows + a GEMM +
 * tb200_token_tail_select_fwd in one pass (tcgen05 MMAs on a CTA pair, the row-wise tail in their epilogue).  Values
 * agree with that three-kernel path to bf16 rounding (the projection is not rounded to bf16 before the SiLU here).
 * tables / table_rows: HOST arrays of n_feat (<= 8) device table pointers (NULL = a feature without a table: zeros)
 * and their row counts; every table is [table_rows[f], emb] bf16; emb in {32, 64, 128}, n_feat * emb in {64, 128}.
 * ids: device int64 [n_feat, rows], clamped into their table.  w: [n_cols, n_feat * emb] bf16 (`nn.Linear.weight`),
 * bias: fp32 [n_cols] or NULL; ln_gamma, ln_beta, rms_gamma: bf16 [n_cols]; table_a / table_b (NULL allowed):
 * bf16 [rows_a / rows_b, n_cols] with device int64 ids per row.  n_cols in {256, 512}; bf16 only.
 * row_dst, rows_out, tokens, normed: as in tb200_token_tail_select_fwd.  status_word: optional device int32 that
 * the kernel sets to 1 if one of its bounded waits gave up (the outputs are then incomplete). */
int tb200_token_project_fwd(const void* const* tables, const int64_t* table_rows, int32_t n_feat, int32_t emb,
                            const int64_t* ids, const void* w, const float* bias, const void* ln_gamma,
                            const void* ln_beta, const void* table_a, int64_t rows_a, const int64_t* ids_a,
                            const void* table_b, int64_t rows_b, const int64_t* ids_b, const void* rms_gamma,
                            const int32_t* row_dst, int64_t rows_out, void* tokens, void* normed, int64_t rows,
                            int32_t n_cols, float ln_eps, float rms_eps, int32_t* status_word, void* stream);

/* ---- (a) sparse-field embedding gather / pool ---------------------------------------------
 * out[b, :] = mean over hot h of table[ids[b, h], :] for ids in (0, vocab_rows); ids equal to 0
 * (padding) or outside the table are skipped; an empty bag gives zeros.  fp32 sum in hot order,
 * one true division by the count, then rounding to `dtype`.  A bag of one id is a bit-exact row copy.
 * Replaces `embedding_bag_mean`
 * (src/taac2026/infrastructure/accelerators/embedding/embedding_bag.py:439-467; oracle
 * `_torch_embedding_bag_mean` :82-83 and the CUDA kernel
 * embedding/kernels/cuembed_embedding_bag_mean.cu:19-47).
 * table: [vocab_rows, dim]; ids: [batch, bag] of `ids_dtype`; out: [batch, dim]. */
int tb200_bag_mean_fwd(const void* table, int64_t vocab_rows, int32_t dim, const void* ids, int ids_dtype,
                       int64_t batch, int32_t bag, void* out, int dtype, void* stream);

/* Sparse gradient of tb200_bag_mean_fwd with respect to the table, in the (row list, value rows) form the reference
 * hands to its sparse optimizer (`SparseEmbeddingBagMean.backward`,
 * src/taac2026/infrastructure/modeling/embeddings.py:34-62; dense atomic form: embedding/kernels/triton.py:105-151):
 *     rows_out[b * bag + h] = ids[b, h],   vals_out[b * bag + h, :] = grad_out[b, :] / (number of valid ids of bag b)
 * for valid ids (0 < id < vocab_rows); the other positions name row 0 and carry zeros, so that the layout is fixed
 * ([batch * bag] rows) and coalescing the list gives the reference's gradient.  No atomics.
 * ids: [batch, bag] of ids_dtype; grad_out: [batch, dim], vals_out: [batch * bag, dim] of `dtype`; rows_out: int64. */
int tb200_bag_mean_bwd(const void* ids, int ids_dtype, const void* grad_out, int64_t* rows_out, void* vals_out,
                       int64_t batch, int32_t bag, int32_t dim, int64_t vocab_rows, int dtype, void* stream);

/* ---- compact host format of the behaviour sequences ------------------------------------------------------------
 * The reference copies padded int64 buffers to the device (ids [B, F, L], timestamps [B, L], lengths [B]; built by
 * `PCVRRecordBatchConverter._build_sequence_inputs`, src/taac2026/infrastructure/data/batch_converter.py:446-488,
 * copied in application/evaluation/workflow.py:246-262).  The compact format holds the valid prefix of every sample
 * in 32 bits:  cu[B + 1] int32 (cu[b] = first event of sample b),  ids[F, ids_stride] int32,  gaps[total] int32 =
 * request_timestamp[b] - timestamp, INT32_MIN where the timestamp is 0.  The tb200_host_* functions run on the host
 * (no CUDA call, usable without a GPU; `threads` worker threads, 1..64); a value that does not fit returns
 * TB200_ERR_RANGE and the caller keeps the padded copy.  tb200_expand_sequence rebuilds the padded int64 tensors on
 * the device bit for bit (positions beyond the length are zero), so the kernels behind see the reference's layout. */

/* cu from the padded record's lengths: cu[b + 1] = cu[b] + clamp(lengths[b], 0, max_len). */
int tb200_host_compact_offsets(const int64_t* lengths, int32_t batch, int32_t max_len, int32_t* cu);

/* Padded int64 record -> compact.  gaps may be NULL (timestamps not carried). */
int tb200_host_compact_sequence(const int64_t* values, const int64_t* timestamps, const int64_t* request_ts,
                                const int32_t* cu, int32_t batch, int32_t feats, int32_t max_len, int32_t* ids,
                                int64_t ids_stride, int32_t* gaps, int32_t threads);

/* Arrow list columns (offsets int32, or int64 with offsets_are_int64; values int64) -> compact, without the padded
 * intermediate: the prefix rule of `pad_list_offsets_values` (batch_converter.py:68-103), length = longest id column
 * (`_fill_sequence`, :503-538), ids <= 0 -> 0 (:476), and with vocab_sizes the clip_vocab=True rule of
 * `_clip_sequence_vocab` / `record_oob` (:594-650) with the clipped ids counted per column in oob_counts (may be
 * NULL).  ts_offsets / ts_values may be NULL (no timestamp column).  Writes cu as well. */
int tb200_host_compact_from_lists(const void* const* id_offsets, const int64_t* const* id_values, int32_t feats,
                                  const void* ts_offsets, const int64_t* ts_values, int32_t offsets_are_int64,
                                  const int64_t* request_ts, const int64_t* vocab_sizes, int64_t* oob_counts,
                                  int32_t batch, int32_t max_len, int32_t* cu, int32_t* ids, int64_t ids_stride,
                                  int32_t* gaps, int32_t threads);

/* The same with the converter's strict time filter (`_fill_strict_sequence`, batch_converter.py:540-592): a row keeps
 * the positions of its timestamp list with 0 < ts < request_ts (the last max_len of them); id columns contribute their
 * values at the kept positions below their own length, compacted to the front.  The timestamp column is required. */
int tb200_host_compact_from_lists_strict(const void* const* id_offsets, const int64_t* const* id_values, int32_t feats,
                                         const void* ts_offsets, const int64_t* ts_values, int32_t offsets_are_int64,
                                         const int64_t* request_ts, const int64_t* vocab_sizes, int64_t* oob_counts,
                                         int32_t batch, int32_t max_len, int32_t* cu, int32_t* ids, int64_t ids_stride,
                                         int32_t* gaps, int32_t threads);

/* Device: compact -> values [B, F, L] int64, lengths [B] int64, timestamps [B, L] int64 (NULL: not written).
 * max_len must be even; values / timestamps 16-byte aligned. */
int tb200_expand_sequence(const int32_t* ids, const int32_t* gaps, const int32_t* cu, const int64_t* request_ts,
                          int64_t* values, int64_t* lengths, int64_t* timestamps, int32_t batch, int32_t feats,
                          int32_t max_len, int64_t ids_stride, void* stream);

/* All sparse fields of one entity in a single launch: the fused form of the per-field Python
 * loop in `FeatureEmbeddingBank.forward`
 * (src/taac2026/infrastructure/modeling/embeddings.py:137-173), including its
 * `.clamp(min=0, max=vocab)` of the raw ids.
 * tables: device array of n_fields table base pointers, each [rows[f], dim] of `dtype`;
 * rows, offsets, lengths: device arrays [n_fields] (table row count; first column and bag size
 * of the field inside one row of `ids`); ids: [batch, ids_cols] of `ids_dtype`;
 * out: [batch, n_fields, dim].  max_bag = max(lengths) (host value, sizes the id staging). */
int tb200_fields_bag_mean_fwd(const void* const* tables, const int64_t* rows, const int32_t* offsets,
                              const int32_t* lengths, int32_t n_fields, int32_t max_bag, int32_t dim, const void* ids,
                              int ids_dtype, int64_t batch, int32_t ids_cols, void* out, int dtype, void* stream);

/* The same with the tokenizer's "missing value" rows folded in (`NonSequentialTokenizer.forward`,
 * src/taac2026/infrastructure/modeling/tokenizers.py:66-68):
 *     out[b, f, :] = pooled[b, f, :] + (missing[b, f] ? missing_rows[f, :] : 0)
 * with the pooled row rounded to `dtype` first and the sum rounded again, i.e. the bits of the two tensor operations
 * `pooled + mask.unsqueeze(-1) * missing_embeddings`.  missing: uint8 / bool flags [batch, missing_cols], of which
 * the first n_fields columns are used; missing_rows: [n_fields, dim] of `dtype`, 16-byte aligned. */
int tb200_fields_bag_mean_missing_fwd(const void* const* tables, const int64_t* rows, const int32_t* offsets,
                                      const int32_t* lengths, int32_t n_fields, int32_t max_bag, int32_t dim,
                                      const void* ids, int ids_dtype, int64_t batch, int32_t ids_cols,
                                      const uint8_t* missing, int32_t missing_cols, const void* missing_rows,
                                      void* out, int dtype, void* stream);

/* out[i, out_col0 : out_col0 + dim] = table[clamp(id_i, 0, vocab_rows - 1), :]   (bit-exact copy)
 * for i in [0, n), with id_i = ids[(i / seq_len) * ids_batch_stride + (i % seq_len)].
 * The `nn.Embedding` gather of `SequenceTokenizer.forward` fused with its id clamp and with the
 * `torch.cat` over features (src/taac2026/infrastructure/modeling/tokenizers.py:156-176): for feature f
 * of a [B, F, L] id tensor pass ids + f * L, seq_len = L, ids_batch_stride = F * L, n = B * L, and
 * out_col0 = f * dim inside output rows of out_stride = F * dim elements.  A flat id vector is
 * seq_len = n, ids_batch_stride = 0.
 * dim, out_col0 and out_stride times sizeof(dtype) must be multiples of 16; table and out 16-byte aligned. */
int tb200_gather_rows(const void* table, int64_t vocab_rows, int32_t dim, const void* ids, int ids_dtype, int64_t n,
                      int64_t seq_len, int64_t ids_batch_stride, void* out, int64_t out_stride, int32_t out_col0,
                      int dtype, void* stream);

/* dst[ids[i], dst_col0 : dst_col0 + dim] = src[i, :] (+ bias[i / rows_per_group, :]) (+ residual[ids[i], :dim])
 * for i in [0, n): the row scatter behind the per-token overrides of OneTrans's non-sequence tokens
 * (`q[:, position, :] = q_proj(token)` and `output[:, position, :] = ffn(...)`,
 * experiments/onetrans/model.py:60-67, :89-93), with the projection bias and the residual stream folded
 * in.  ids: device int64[n], distinct rows of dst; src [n, dim] dense; bias [n / rows_per_group, dim] or
 * NULL; residual rows of residual_stride elements or NULL (may alias dst only if dst_col0 == 0 and the
 * strides agree, since every row is read before it is written by the same thread).  dim, dst_col0 and
 * the strides times sizeof(dtype) must be multiples of 16. */
int tb200_scatter_rows(void* dst, int64_t dst_rows, int64_t dst_stride, int32_t dst_col0, const int64_t* ids,
                       const void* src, int64_t n, int32_t dim, const void* bias, int64_t rows_per_group,
                       const void* residual, int64_t residual_stride, int dtype, void* stream);

/* x[i, :] = x[i, :] + table_a[ids_a[i], :], then (table_b != NULL) + table_b[ids_b[i], :], in place; ids are
 * clamped into their table and every sum is rounded to `dtype` like a tensor addition of its own.  The
 * sequence tokenizer's `tokens = tokens + self.time_embedding(time_values)`
 * (src/taac2026/infrastructure/modeling/tokenizers.py:188-189) and the sinusoidal position rows added by
 * the experiment model, without materialising the gathered rows.  x: [n, dim]; ids: device int64[n];
 * dim * sizeof(dtype) a multiple of 16. */
int tb200_add_gathered_rows(void* x, int64_t n, int32_t dim, const void* table_a, int64_t rows_a, const int64_t* ids_a,
                            const void* table_b, int64_t rows_b, const int64_t* ids_b, int dtype, void* stream);

/* x[r, :] = act(x[r, :] + bias[r / rows_per_group, :]) in place; act 0 = identity, 1 = SiLU with the sum
 * rounded to `dtype` before the activation: the `nn.Linear` bias (+ `nn.SiLU()`) of OneTrans's per-token
 * projections and `FeedForward` (experiments/onetrans/model.py:36-41, :60-67) when the linear parts of all
 * tokens run as one batched product.  x: [rows, cols]; bias: [rows / rows_per_group, cols];
 * cols * sizeof(dtype) a multiple of 16. */
int tb200_bias_act_rows(void* x, int64_t rows, int32_t cols, const void* bias, int64_t rows_per_group, int32_t act,
                        int dtype, void* stream);

/* ---- (c) varlen masked attention forward ----------------------------------------------------
 * o[b, h, q, :] = softmax_k(scale * <q[b, h, q, :], k[b, h, k, :]> over visible k) . v[b, h, k, :]
 * with fp32 softmax statistics and accumulation.  Key k is visible to query q of sample b iff
 *     (k < seq_len[b]  or  k >= ns_start)  and  k < Lk  and  (not causal or k <= q).
 * With padded_query_self, queries in [seq_len[b], ns_start) return v[b, h, q, :] (needs Lq == Lk);
 * a query without any visible key returns zeros.  The mask is never materialised.
 * Replaces the inference branch of `flash_attention`
 * (src/taac2026/infrastructure/accelerators/attention/flash_attention.py:871-919; mask planner
 * :149-198 -> (seq_len, causal, padded_query_self); self fallback :201-209; kernel
 * attention/kernels/tilelang.py:36-138; oracle `_torch_flash_attention` :552-570).  ns_start extends
 * the planner's two mask families to OneTrans's [sequence | always-valid NS tokens] layout
 * (experiments/onetrans/model.py:325-330); ns_start >= Lk means no such suffix.
 * strides: 12 host values, in elements: (batch, head, row) for q, k, v, o; the head dim is contiguous
 * and every stride a multiple of 8.  seq_len: device int32[B] or NULL (all keys valid).
 * cu_rows: device int32[B + 1] or NULL; when given, the batch is packed along the row axis: sample b
 * owns rows [cu_rows[b], cu_rows[b+1]) (batch strides and seq_len unused, every key valid, Lq and Lk
 * are upper bounds of any sample's row count).
 * cu_rows_q: device int32[B + 1] or NULL (needs cu_rows): q and o are packed by these offsets instead;
 * sample b's lq = cu_rows_q[b+1] - cu_rows_q[b] queries are the LAST lq of its lk rows, so the causal rule
 * becomes k <= q + (lk - lq).  This is the block of OneTrans's pyramid (experiments/onetrans/model.py:340-348
 * keeps `sequence_part[:, -keep_count:]` after the block) evaluated for the kept rows only; Lq then bounds
 * the query counts, Lk the key counts.  Served by kernels 1, 3 and 4; the automatic choice is 3 up to 32
 * rows and 4 beyond (D = 64), else 1.
 * key_valid: device uint8[B, Lk] or NULL; when given it replaces the (seq_len, ns_start) rule by
 * "key k is valid iff key_valid[b, k] != 0" for arbitrary padding patterns (several sequence domains
 * with separators, experiments/onetrans/model.py:287-315); padded queries are the invalid positions.
 * D in {32, 64, 128}; dtype TB200_BF16 or TB200_F16.  dtype TB200_F32 (any D <= 256 that is a multiple of 4, at
 * most 8192 keys per sample, strides multiples of 4) selects a plain fp32 kernel — every product, the softmax and
 * the weighted sum in fp32, one warp per query row — for comparing an fp32 model with the reference's fp32 torch
 * path (`_torch_flash_attention`, flash_attention.py:552-570); it ignores `kernel` and is not a serving kernel.
 * kernel: 0 = automatic, 1 = mma.sync kernel (every supported shape), 2 = tcgen05/TMEM kernel (D = 64, bf16,
 * no key_valid map; TB200_ERR_UNSUPPORTED otherwise), 3 = one warp per (sample, head) (D = 64, at most 32
 * rows), 4 = one warp per (sample, head) streaming the keys in tiles of 16 against 16 queries in registers
 * (packed batches, D = 64: few queries, many keys).  total_rows: row count of the packed matrices when
 * cu_rows is given (bounds the TMA tensor maps), ignored otherwise.  status_word: optional device int32 that
 * the tcgen05 kernel sets to 1 if one of its bounded waits gave up. */
int tb200_attn_fwd(const void* q, const void* k, const void* v, void* o, int32_t B, int32_t H, int32_t Lq,
                   int32_t Lk, int32_t D, const int64_t* strides, const int32_t* seq_len, const int32_t* cu_rows,
                   const int32_t* cu_rows_q, const uint8_t* key_valid, int32_t ns_start, int32_t causal, int32_t padded_query_self, float scale, int dtype,
                   int32_t kernel, int64_t total_rows, int32_t* status_word, void* stream);

/* Attention backward for the padded (B, H, L, D) layout: dq, dk, dv from q, k, v, o and the upstream gradient d_o,
 * under the same mask arguments as tb200_attn_fwd (no packed batches).  First, plain form of the reference's
 * `flash_attention_backward` (accelerators/attention/kernels/tilelang.py:440-701; preprocess :395-437): fp32 arithmetic,
 * scores recomputed, two kernels (per query row, per key row), no atomics.  strides: the 12 values of tb200_attn_fwd;
 * d_o uses o's strides, dq / dk / dv those of q / k / v.  workspace: tb200_attn_bwd_workspace_bytes(B, H, Lq) bytes
 * of device memory (log-sum-exp and dO.O per query row).  D <= 256, Lq, Lk <= 4096; fp32, fp16 or bf16. */
int64_t tb200_attn_bwd_workspace_bytes(int32_t B, int32_t H, int32_t Lq);
int tb200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, void* dq, void* dk,
                   void* dv, void* workspace, int32_t B, int32_t H, int32_t Lq, int32_t Lk, int32_t D,
                   const int64_t* strides, const int32_t* seq_len, const uint8_t* key_valid, int32_t ns_start,
                   int32_t causal, int32_t padded_query_self, float scale, int dtype, void* stream);

/* ---- (d) FP8 e4m3 block-scaled FFN ---------------------------------------------------------
 * The reference has no FP8 path: its FFNs are bf16/fp32 torch modules — the SiLU-gated
 * `down(silu(gate) * value)` of experiments/tokenformer/model.py:118-128 and
 * experiments/symbiosis/backbone.py:11-21, and OneTrans's ungated `Linear -> SiLU -> Linear`
 * (experiments/onetrans/model.py:33-44).  These entry points compute the same layers with e4m3
 * operands: activations carry one fp32 scale per 1 x 128 block of a row, weights one per
 * 128 x 128 block, both scale = amax / 448 (1 where amax == 0), value = e4m3 * scale.
 *
 * x_bf16 [M, K] -> x_fp8 [M, K] e4m3, scales [M, K / 128].  K % 128 == 0. */
int tb200_quant_act_1x128(const void* x_bf16, void* x_fp8, float* scales, int64_t M, int32_t K, void* stream);

/* out = epilogue( dequant(a) @ dequant(b)^T ), a: [M, K] e4m3 with a_scales [M, K / 128],
 * b: [N, K] e4m3 (a torch Linear weight) with b_scales [N / 128, K / 128]; fp32 accumulation,
 * every 128-wide K block scaled by its own (a, b) scale pair.  N % 256 == 0, K % 128 == 0.
 * mode 0 (SiLU-gated): b's rows are interleaved per 128-column hidden block t as
 *        [gate rows of block t | value rows of block t]; out = e4m3 [M, N / 2] of silu(gate) * value,
 *        out_scales [M, N / 256]; bias (optional, fp32 [N]) in the same interleaved order.
 * mode 1 (SiLU):       out = e4m3 [M, N] of silu(acc + bias), out_scales [M, N / 128].
 * mode 2 (linear):     out = bf16 [M, N] of acc + bias (+ residual bf16 [M, N]); out_scales unused.
 * bias and residual may be NULL.  status_word: optional device int32 that the kernel sets to 1 if
 * one of its bounded waits gave up (the output is then incomplete). */
int tb200_fp8_gemm(const void* a_fp8, const float* a_scales, const void* b_fp8, const float* b_scales,
                   const float* bias, const void* residual, void* out, float* out_scales, int64_t M, int32_t N,
                   int32_t K, int32_t mode, int32_t* status_word, void* stream);

/* ---- FP8 FFN with power-of-two (UE8M0) block scales applied by the tensor cores --------------------------------
 * Same block structure as above (1 x 128 activation blocks, 128 x 128 weight blocks, scales derived from the block's
 * amax), but the scale is rounded up to a power of two and multiplied in by `tcgen05.mma.kind::mxf8f6f4.block_scale`,
 * so a tile accumulates over the whole K in tensor memory and the epilogue runs once per tile.  No counterpart in the
 * reference (it has no FP8 path); serves the FFN modules of experiments/onetrans/model.py:33-44 and
 * experiments/tokenformer/model.py:118-128.
 * Scale factors are stored as 512-byte atoms per (128 rows, 128-wide K block): byte (r % 32) * 16 + (r / 32) * 4 + s is
 * the exponent byte (value 2^(byte - 127)) of row r, 32-wide slice s.  Activations: [ceil(M / 128), K / 128, 512];
 * weights: [N / 128, K / 128, 512]; tb200_mx_scale_bytes(rows, K) gives the size.  Atom arrays should be zeroed
 * before first use when M is not a multiple of 128 (rows beyond M are never written). */
int64_t tb200_mx_scale_bytes(int64_t rows, int32_t K);
/* bf16 [M, K] -> e4m3 [M, K] + activation scale atoms. */
int tb200_quant_act_mx(const void* x_bf16, void* x_fp8, uint8_t* scale_atoms, int64_t M, int32_t K, void* stream);
/* out = epilogue(a @ b^T): mode 0 = SiLU-gated ([128 gate | 128 value] rows per 256-row weight tile) -> e4m3 hidden
 * [M, N / 2] + its scale atoms; 1 = SiLU -> e4m3 hidden [M, N] + atoms; 2 = bias (+ residual) -> bf16 [M, N].
 * N % 256 == 0, K % 128 == 0, K <= 8192; every pointer 16-byte aligned. */
int tb200_mx_gemm(const void* a_fp8, const uint8_t* a_scale_atoms, const void* b_fp8, const uint8_t* b_scale_atoms,
                  const float* bias, const void* residual, void* out, uint8_t* out_scale_atoms, int64_t M, int32_t N,
                  int32_t K, int32_t mode, int32_t* status_word, void* stream);

/* ---- integer sequence preprocessing ---------------------------------------------------------
 * Per sample of one sequence domain: which events survive duplicate removal, and the six sequence
 * statistics.  Replaces `deduplicate_sequence_events`
 * (src/taac2026/infrastructure/modeling/sequence.py:141-198) and `compute_sequence_stats`
 * (src/taac2026/infrastructure/modeling/time_features.py:49-105), bit for bit.
 * values [batch, n_feat, max_len], lengths [batch], timestamps [batch, max_len], request_ts [batch], all int64.
 * out_len [batch] int64: length after duplicate removal (the input length for untouched samples);
 * out_src [batch, max_len] int32: source position of every output slot (identity for untouched samples,
 *   -1 for the zero-filled tail of changed samples) — new_values[b, f, j] = values[b, f, out_src[b, j]];
 * out_stats [batch, 6] fp32: [length, active, distinct, 1 - distinct / active, positive share, last gap bucket].
 * The statistics always describe the INPUT (before removal).  max_len <= 8192. */
int tb200_sequence_prepare(const int64_t* values, const int64_t* lengths, const int64_t* timestamps,
                           const int64_t* request_ts, int64_t batch, int32_t n_feat, int32_t max_len,
                           int64_t* out_len, int32_t* out_src, float* out_stats, void* stream);

/* Index vectors of the packed valid-token layout: for every row of the packed token matrix the ids of
 * `SequenceTokenizer.forward`'s embedding lookups (src/taac2026/infrastructure/modeling/tokenizers.py:156-176;
 * hashed like `modeling/embeddings.py:74-79` where a table is a compressed one), the position inside the
 * cropped sequence (`modeling/sequence.py:130-138` indexes the sinusoidal table with it) and the time-gap
 * bucket (`modeling/time_features.py:31-46`), after duplicate removal and tail crop.
 * Sample b owns rows [cu_rows[b], cu_rows[b+1]): seq_count[b] sequence tokens, then its non-sequence tokens
 * (their entries are 0).  Sequence token j is input position src[b, start[b] + j], src = out_src of
 * tb200_sequence_prepare.  hash_buckets [n_feat]: 0 = raw ids, > 0 = ((v - 1) mod buckets) + 1 for v > 0 else 0,
 * < 0 = feature without a table (its ids are not written).  ids_out [n_feat, total_rows], pos_out and
 * bucket_out [total_rows] int64; bucket_out (with timestamps / edges) may be NULL.  All inputs int64 on the
 * device except src (int32). */
int tb200_packed_token_index(const int64_t* values, const int64_t* timestamps, const int64_t* request_ts,
                             const int32_t* src, const int64_t* cu_rows, const int64_t* seq_count, const int64_t* start,
                             const int64_t* edges, int32_t n_edges, const int64_t* hash_buckets, int64_t batch,
                             int32_t n_feat, int32_t max_len, int64_t total_rows, int64_t* ids_out, int64_t* pos_out,
                             int64_t* bucket_out, void* stream);

/* Row plan of the packed valid-token layout for a whole forward, in one launch.  widths[0 .. n_layers] (host array)
 * is the static pyramid schedule of padded sequence widths (`_pyramid_keep_count`, experiments/onetrans/model.py:
 * 317-323; widths[0] = min(max_len, seq_top_k)); lengths: [batch] int64 after duplicate removal.  Outputs (device):
 *   start[b] = max(raw - widths[0], 0), n0[b] = min(raw, widths[0]) with raw = clamp(lengths[b], 0, max_len)
 *   counts[l, b] = max(n0[b] - (widths[0] - widths[l]), 0)          valid sequence tokens of sample b at layer l
 *   cu[l, 0 .. batch] / cu32[l, ...]   exclusive prefix sums of counts[l, :] + ns (int64 and int32 copies)
 *   meta[l] = (total rows, largest rows per sample) of layer l       the one pair of numbers per layer the host reads
 *   ns_rows0[b, j] = cu[0, b] + counts[0, b] + j                     rows of the non-sequence tokens at layer 0
 * These are the integers behind `tokens[:, -keep_count:]` (model.py:340-348) when only valid tokens are stored.
 * n_layers <= 64, (widths[0] + ns) * batch < 2^31. */
int tb200_pyramid_plan(const int64_t* lengths, int32_t batch, int32_t max_len, const int32_t* widths, int32_t n_layers,
                       int32_t ns, int64_t* start, int64_t* n0, int64_t* counts, int64_t* cu, int32_t* cu32,
                       int64_t* meta, int64_t* ns_rows0, void* stream);

/* Rows of layer l kept for layer l + 1, from two consecutive rows of the plan above (cu0 = cu[l], cu1 = cu[l + 1], ...):
 * src[cu1[b] + r] = cu0[b] + (counts0[b] - counts1[b]) + r;  ns_rows1[b, j] = cu1[b] + counts1[b] + j;  row_dst
 * (optional, int32 [rows of layer l]) = the destination of every row of layer l, -1 for the dropped ones. */
int tb200_pyramid_kept_rows(const int64_t* cu0, const int64_t* cu1, const int64_t* counts0, const int64_t* counts1,
                            int32_t batch, int32_t ns, int64_t* src, int64_t* ns_rows1, int32_t* row_dst, void* stream);

/* ---- per-token (grouped) bf16 linear layers with a fused epilogue ----------------------------
 * out[g] = act(a[g] @ w[g]^T + bias[g]) (+ residual[g]) for g in [0, groups): the token-specific projections
 * and feed-forward layers of the non-sequence tokens, `nn.ModuleList` of `nn.Linear` / `FeedForward` applied
 * token by token (experiments/onetrans/model.py:137-147 `_ns_linear`, :160-166 the `ns_specific` FFNs), which
 * a batched library GEMM plus separate bias / SiLU / residual passes would otherwise serve.
 * a: [groups, M, K], w: [groups, N, K] (stacked `nn.Linear.weight`), out and residual: [groups, M, N], all
 * bf16 and contiguous; bias: fp32 [groups, N]; bias and residual may be NULL; residual may be `out` itself.
 * act: 0 = none, 1 = SiLU, 2 = SiLU-gated: the N rows of w[g] are interleaved per 128 hidden columns as
 * [128 gate rows | 128 value rows] (the order tb200_fp8_gemm's mode 0 takes, bias likewise), out is
 * [groups, M, N / 2] = silu(gate) * value — the first half of `down(silu(gate) * value)`
 * (experiments/tokenformer/model.py:118-128) on the bf16 tensor cores; no residual with act 2.
 * fp32 accumulation over the whole K, one rounding to bf16 at the end.
 * N % 256 == 0, K % 64 == 0.  groups = 1 is a plain linear layer.  status_word: optional device int32 that the
 * kernel sets to 1 if one of its bounded waits gave up (the output is then incomplete). */
int tb200_gemm_bf16_grouped(const void* a, const void* w, const float* bias, const void* residual, void* out,
                            int32_t groups, int64_t M, int32_t N, int32_t K, int32_t act, int32_t* status_word,
                            void* stream);

/* ---- whole FFN without any allocation --------------------------------------------------------
 * No counterpart in the reference (which has neither an FP8 path nor a C interface).
 *
 * y = [residual +] W_down . act(W_up . x + b_up) + b_down for bf16 x [M, d_in], i.e. the three calls
 * tb200_quant_act_1x128 -> tb200_fp8_gemm(mode 0 if gated else 1) -> tb200_fp8_gemm(mode 2) in one
 * entry point that needs no workspace from the caller.  It exists for callers that cannot allocate
 * device memory at the point where they run the layer: code inside a serving loop whose memory was
 * handed out once at start-up and is fully committed, a plugin called from a host framework that
 * owns the allocator, or a latency-critical path where a cudaMalloc (which synchronises the device)
 * is not acceptable.  Such a caller still passes x, the prepared weights and y; the quantised input,
 * the e4m3 hidden activation and their scales live in a fixed array inside the library.
 *
 * Limits and rules:
 *  - the array is tb200_ffn_fp8_static_scratch_bytes() = 64 MiB per GPU, held from library load to
 *    process exit; a call needs about M * (d_in + hidden) * 1.04 bytes (d_in 512, hidden 2048:
 *    M <= 25 000 rows).  Larger requests return TB200_ERR_SCRATCH and launch nothing — split the rows;
 *  - the first call on each device looks the array's address up (cudaGetSymbolAddress) and sets kernel
 *    attributes; make that call once per device before capturing a stream or timing anything;
 *  - the entry point calls no cudaMalloc / cudaFree and no allocating library routine;
 *  - every call on a device uses the same array: two calls that overlap on the GPU (different streams,
 *    or graphs replayed concurrently) race on it.  Calls on one stream are ordered and safe.  Nothing
 *    in the data part of the array needs clearing between calls: each call overwrites all bytes it later
 *    reads.  The array's first word is a status word: the call clears it (a 4-byte memset on `stream`) and
 *    the two GEMM kernels set it to 1 if one of their bounded waits gave up — read it with
 *    tb200_ffn_fp8_static_status;
 *  - every argument check of the three steps is made before the first launch: a negative return value
 *    means that nothing was enqueued.
 * w_up_fp8 / w_up_scales / b_up and w_down_* are exactly what the two tb200_fp8_gemm calls take
 * (for gated != 0 the [gate | value] row interleave of mode 0); b_up, b_down and residual may be NULL.
 * d_in % 128 == 0, hidden % 256 == 0, d_out % 256 == 0. */
int tb200_ffn_fp8_fwd_static(const void* x_bf16, const void* w_up_fp8, const float* w_up_scales, const float* b_up,
                             const void* w_down_fp8, const float* w_down_scales, const float* b_down,
                             const void* residual, void* y_bf16, int64_t M, int32_t d_in, int32_t hidden,
                             int32_t d_out, int32_t gated, void* stream);

/* Size in bytes of the fixed array behind tb200_ffn_fp8_fwd_static. */
int64_t tb200_ffn_fp8_static_scratch_bytes(void);

/* Status word of the calls to tb200_ffn_fp8_fwd_static enqueued on `stream` so far (current device):
 * *value = 0 if every kernel of the last call ran to completion, 1 if a bounded wait inside one of them
 * gave up (y is then incomplete).  Copies four bytes to the host and SYNCHRONISES `stream`; allocates
 * nothing.  No counterpart in the reference. */
int tb200_ffn_fp8_static_status(void* stream, int32_t* value);

#ifdef __cplusplus
}
#endif

#endif /* TB200_H_ */
