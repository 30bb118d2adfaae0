/*
 * darkforest_kernels.h — C ABI of the B200 (sm_100a) fused causal attention library.
 *
 * Drop-in boundary: every extern "C" symbol of darkforest-cuda/kernels/attention_fused.cu is
 * exported here with the exact name and signature that Dark Forest's Rust FFI shim binds, so
 * darkforest-cuda/src/kernels.rs links unchanged. The training path (the hot path):
 *   launch_fused_attention     replaces darkforest-cuda/kernels/attention_fused.cu:223-231
 *                              (bound at darkforest-cuda/src/kernels.rs:706-716)
 *   launch_fused_mha_forward   replaces attention_fused.cu:233-242   (kernels.rs:802-812)
 *   launch_attention_backward  replaces attention_fused.cu:361-378   (kernels.rs:752-765)
 *   launch_fused_mha_backward  replaces attention_fused.cu:518-532   (kernels.rs:850-864)
 *   darkforest_sync            replaces darkforest-cuda/kernels/matmul.cu:21-28
 *                              (bound at kernels.rs:9-20)
 * and, declared further down with their own notes, the decode family (launch_fused_mha_decode_kv,
 * _splitk, launch_paged_mha_decode_kv, _splitk, _bf16) and the per-token helpers
 * (launch_apply_rope, launch_pos_embed_interpolate, launch_paged_copy_row, _f32_to_bf16).
 *
 * Contract shared by every entry point:
 *   - all pointers are caller-owned DEVICE memory; nothing is allocated or freed per call;
 *   - tensors are row-major [S, H*D] fp32, head h = columns h*D..(h+1)*D-1
 *     (attention_fused.cu:60-66); a batch is B contiguous slabs [B][S][H*D];
 *   - O, dQ, dK, dV (and lse, delta where present) are fully overwritten, never accumulated
 *     (the reference memsets dK/dV and overwrites dQ: attention_fused.cu:522-524, 510-515);
 *   - inputs must not alias outputs; any S >= 0, 1 <= D <= 128, causal or not;
 *   - launches are asynchronous. Legacy symbols use the legacy default stream as the
 *     reference does (attention_fused.cu:229,240,375,529); df_* symbols take a stream;
 *   - no entry point aborts or traps: arguments are validated on the host, the legacy
 *     void symbols record a sticky per-thread status readable with df_attn_last_status().
 */
#ifndef DARKFOREST_KERNELS_H
#define DARKFOREST_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define DF_API __attribute__((visibility("default")))
#else
#define DF_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (df_* return value, df_attn_last_status) ---- */
#define DF_OK 0
#define DF_ERR_INVALID_ARG 1   /* null pointer, D outside 1..128, size overflow            */
#define DF_ERR_UNSUPPORTED 2   /* a shape the selected variant cannot run                   */
#define DF_ERR_CUDA 3          /* a CUDA runtime/driver call failed                         */
#define DF_ERR_DEVICE_TIMEOUT 4 /* a bounded wait inside a kernel ran out (see df_sync_status) */
#define DF_ERR_WORKSPACE 5     /* caller scratch too small                                  */
#define DF_ERR_STATIC_SCRATCH 6 /* problem larger than the library's built-in scratch array  */
#define DF_ERR_RING_TIMEOUT 7  /* darkforest_ring.h: a host-side wait on the communicator ran out; it was aborted */
#define DF_ERR_NCCL 8          /* darkforest_ring.h: NCCL reported an error (df_ring_last_nccl_result)          */
#define DF_ERR_DEVICE_BOUNDS 9 /* DF_BOUNDS_CHECK builds only: a kernel computed an index outside its tensor (see df_sync_status) */

/* ---- legacy symbols: signatures identical to the reference ---- */

/* Single-head forward on [S, D]. Reference: attention_fused.cu:223-231. */
DF_API void launch_fused_attention(const float *q, const float *k, const float *v, float *out,
                            uint32_t seq_len, uint32_t d_head, float scale, uint32_t causal);

/* Multi-head forward on [S, H*D]. Reference: attention_fused.cu:233-242. */
DF_API void launch_fused_mha_forward(const float *q, const float *k, const float *v, float *out,
                              uint32_t n_heads, uint32_t seq_len, uint32_t d_head, float scale,
                              uint32_t causal);

/* Single-head backward. `probabilities` is caller scratch of at least S*S floats
 * (darkforest-cuda/src/lib.rs:2431-2479); its contents are undefined afterwards.
 * Reference: attention_fused.cu:361-378. */
DF_API void launch_attention_backward(const float *q, const float *k, const float *v, const float *d_out,
                               float *d_q, float *d_k, float *d_v, float *probabilities,
                               uint32_t seq_len, uint32_t d_head, float scale, uint32_t causal);

/* Multi-head backward. `probabilities` is caller scratch of at least H*2*S*S floats
 * (darkforest-cuda/src/lib.rs:2019-2027). Reference: attention_fused.cu:518-532. */
DF_API void launch_fused_mha_backward(const float *q, const float *k, const float *v, const float *d_out,
                               float *d_q, float *d_k, float *d_v, float *probabilities,
                               uint32_t n_heads, uint32_t seq_len, uint32_t d_head, float scale,
                               uint32_t causal);

/* ---- Decode: one query token per head against a KV cache (legacy symbols, same signatures) ----
 * q, out: [n_heads * d_head] fp32. Contiguous cache: k_cache, v_cache [max_seq_len, n_heads * d_head]
 * fp32, the first cur_seq_len rows are attended. Paged cache: k_pool, v_pool are pools of pages of
 * page_size rows, token t lives in row t % page_size of page block_table[t / page_size].
 * cur_seq_len == 0 leaves `out` untouched, like the reference. Launched on the legacy stream.
 *   launch_fused_mha_decode_kv         replaces attention_fused.cu:617-626  (kernels.rs:1157-1190)
 *   launch_fused_mha_decode_kv_splitk  replaces attention_fused.cu:762-788  (kernels.rs:1254-1303)
 *   launch_paged_mha_decode_kv         replaces attention_fused.cu:1028-1043 (kernels.rs:1307-1350)
 *   launch_paged_mha_decode_kv_splitk  replaces attention_fused.cu:1045-1073
 *   launch_paged_mha_decode_kv_bf16    replaces attention_fused.cu:1075-1090 (pool elements are bf16)
 * The split-K forms take caller scratch for ceil(cur_seq_len / chunk_size) partial states per
 * head: partial_m, partial_l [n_heads * chunks], partial_o [n_heads * chunks * d_head]; this
 * library splits every call over many CTAs anyway and uses at most that many states (contents
 * undefined afterwards). The forms without scratch merge through distributed shared memory. */
DF_API void launch_fused_mha_decode_kv(const float *q, const float *k_cache, const float *v_cache, float *out,
                                uint32_t n_heads, uint32_t cur_seq_len, uint32_t d_head, float scale);
DF_API void launch_fused_mha_decode_kv_splitk(const float *q, const float *k_cache, const float *v_cache,
                                       float *partial_m, float *partial_l, float *partial_o, float *out,
                                       uint32_t n_heads, uint32_t cur_seq_len, uint32_t d_head, float scale,
                                       uint32_t chunk_size);
DF_API void launch_paged_mha_decode_kv(const float *q, const float *k_pool, const float *v_pool,
                                const int32_t *block_table, float *out, uint32_t n_heads,
                                uint32_t cur_seq_len, uint32_t d_head, float scale, uint32_t page_size);
DF_API void launch_paged_mha_decode_kv_splitk(const float *q, const float *k_pool, const float *v_pool,
                                       const int32_t *block_table, float *partial_m, float *partial_l,
                                       float *partial_o, float *out, uint32_t n_heads, uint32_t cur_seq_len,
                                       uint32_t d_head, float scale, uint32_t page_size, uint32_t chunk_size);
DF_API void launch_paged_mha_decode_kv_bf16(const float *q, const void *k_pool, const void *v_pool,
                                     const int32_t *block_table, float *out, uint32_t n_heads,
                                     uint32_t cur_seq_len, uint32_t d_head, float scale, uint32_t page_size);

/* All decode forms in one call, with a status and a stream. block_table NULL: contiguous cache.
 * partial_* NULL (or max_chunks < 2): scratch-free form; otherwise at most max_chunks partial
 * states per head are used. kv_bf16 != 0: k, v point at bf16 elements. */
DF_API int df_attn_decode(const float *q, const void *k, const void *v, const int32_t *block_table, float *out,
                   float *partial_m, float *partial_l, float *partial_o, uint32_t max_chunks,
                   uint32_t n_heads, uint32_t cur_seq_len, uint32_t d_head, float scale,
                   uint32_t page_size, uint32_t kv_bf16, void *stream);

/* ---- The per-token helpers of the same reference file (legacy symbols, legacy stream) ----
 *   launch_pos_embed_interpolate       replaces attention_fused.cu:1127-1139: out[d_model] = row `pos` of the
 *       trained table, or, when max_ctx_len > trained_ctx_len (or pos >= trained_ctx_len), the linear
 *       interpolation at pos * (trained-1)/(max-1). Rejected here instead of reading out of bounds:
 *       max_ctx_len < 2 or pos >= max_ctx_len in the stretched form.
 *   launch_apply_rope                  replaces attention_fused.cu:1168-1177: rotates pairs (2i, 2i+1) of every
 *       head of one row [n_heads * d_head] in place by pos * base_freq^(-2i/d_head). The frequency is
 *       evaluated in double and rounded once (the reference uses powf).
 *   launch_paged_copy_row              replaces attention_fused.cu:1196-1207: pool row
 *       phys_block * page_size + page_offset <- src[d_model].
 *   launch_paged_copy_row_f32_to_bf16  replaces attention_fused.cu:1223-1231: same into a bf16 pool (RNE).
 *   df_attn_apply_rope_rows            batched form without reference counterpart: `rows` consecutive rows,
 *       row r at position first_pos + r, on a stream, with a status. */
DF_API void launch_pos_embed_interpolate(const float *pos_table, float *out, uint32_t pos, uint32_t trained_ctx_len,
                                  uint32_t max_ctx_len, uint32_t d_model);
DF_API void launch_apply_rope(float *qk, uint32_t pos, uint32_t n_heads, uint32_t d_head, float base_freq);
DF_API void launch_paged_copy_row(const float *src, float *pool, int32_t phys_block, uint32_t page_offset,
                           uint32_t page_size, uint32_t d_model);
DF_API void launch_paged_copy_row_f32_to_bf16(const float *src, void *pool, int32_t phys_block, uint32_t page_offset,
                                       uint32_t page_size, uint32_t d_model);
DF_API int df_attn_apply_rope_rows(float *qk, uint32_t first_pos, uint32_t rows, uint32_t n_heads, uint32_t d_head,
                            float base_freq, void *stream);

/* Host-only probe of the explicit work lists that the persistent kernels receive when the round-robin
 * order would leave a heavy tail (up to 2048 items): first-fit decreasing under a binary-searched
 * capacity. Fills off[grid + 1] and items[n] (CTA c runs items[off[c] .. off[c+1]) in that order) and
 * returns 1, or returns 0 when no table is used (n <= grid, n > 2048, grid > 160, or nothing better than
 * the round-robin order was found). No counterpart in the reference. */
DF_API int df_attn_schedule_build(const uint32_t *weights, int n, int grid, uint16_t *off, uint16_t *items);

/* Sizes in bytes of the caller-owned scratch and statistics buffers (host only, nothing is allocated
 * here; no counterpart in the reference, which sizes its one scratch buffer in lib.rs:2019-2027).
 * seq_len is the sequence length, or the cache length for DF_WS_DECODE_PARTIALS (chunk_size as in the
 * split-K decode calls; ignored by the other kinds). Unknown kind: 0. */
#define DF_WS_DELTA 0
#define DF_WS_LSE 1
#define DF_WS_LEGACY_BACKWARD 2
#define DF_WS_LEGACY_BACKWARD_MIN 3
#define DF_WS_DECODE_PARTIALS 4
DF_API uint64_t df_attn_workspace_bytes(int kind, uint32_t batch, uint32_t n_heads, uint32_t seq_len, uint32_t d_head,
                                 uint32_t chunk_size);

/* Host-side view of the static work distribution of the persistent kernels (no GPU involved; no
 * counterpart in the reference): the index of the work item that CTA `cta` of `grid` processes in
 * round `round` when `n_items` items are numbered heaviest first, or -1 past the end of its list. */
DF_API long long df_attn_schedule_item(int round, int grid, int cta, long long n_items);

/* cudaDeviceSynchronize. The reference prints and abort()s on error (matmul.cu:21-28); this
 * one records the status (df_attn_last_status) and returns. */
DF_API void darkforest_sync(void);

/* ---- extended entry points (stream-aware, batched, logsumexp-saving) ---- */

/* Forward: out [B,S,H*D], lse [B,H,S] (natural log; may be NULL).
 * Extends launch_fused_mha_forward (attention_fused.cu:233-242) with batch, lse and stream. */
DF_API int df_attn_forward(const float *q, const float *k, const float *v, float *out, float *lse,
                    uint32_t batch, uint32_t n_heads, uint32_t seq_len, uint32_t d_head,
                    float scale, uint32_t causal, void *stream);

/* Forward of one block of a larger attention problem (ring / sequence-parallel step):
 * queries [B,Sq,H*D] against keys/values [B,Sk,H*D]; key j is visible to query i iff
 * !causal or j <= i + causal_shift (causal_shift = q_global_offset - k_global_offset).
 * Rows with no visible key produce out = 0, lse = -inf
 * (the reference's l > 0 guard, attention_fused.cu:104). */
DF_API int df_attn_forward_block(const float *q, const float *k, const float *v, float *out, float *lse,
                          uint32_t batch, uint32_t n_heads, uint32_t seq_q, uint32_t seq_k,
                          uint32_t d_head, float scale, uint32_t causal, int64_t causal_shift,
                          void *stream);

/* bf16 variant of df_attn_forward_block: q, k, v, out hold bf16 elements (same [B,S,H*D] layout,
 * 2 bytes per element, 16-byte aligned), lse stays fp32. MMAs are kind::f16 with bf16 operands and
 * fp32 accumulation; P is rounded to bf16 before the PV product. d_head must be 64 or 128 (other
 * shapes return DF_ERR_UNSUPPORTED: the bf16 variant has no SIMT fallback). No counterpart in the
 * reference, whose attention is fp32 only (attention_fused.cu:41-159). */
DF_API int df_attn_forward_bf16(const void *q, const void *k, const void *v, void *out, float *lse,
                         uint32_t batch, uint32_t n_heads, uint32_t seq_q, uint32_t seq_k,
                         uint32_t d_head, float scale, uint32_t causal, int64_t causal_shift,
                         uint32_t out_fp32, void *stream);
/* out_fp32 != 0: `out` receives fp32 elements instead of bf16 (ring steps merge partial results in fp32). */

/* bf16 variant of df_attn_backward: q, k, v, out, d_out and the gradients d_q, d_k, d_v hold bf16
 * elements; lse and the delta scratch [B,H,S] stay fp32. d_head 64 or 128 only. P and dS are
 * rounded to bf16 before the gradient products; accumulation is fp32. No reference counterpart. */
DF_API int df_attn_backward_bf16(const void *q, const void *k, const void *v, const void *out, const void *d_out,
                          const float *lse, void *d_q, void *d_k, void *d_v, float *delta, uint32_t batch,
                          uint32_t n_heads, uint32_t seq_len, uint32_t d_head, float scale, uint32_t causal,
                          void *stream);

/* Pieces of the bf16 backward for ring steps: the delta pre-pass on bf16 out / d_out, and the block form
 * (separate seq_q / seq_k, causal shift, final lse and delta given). With out_fp32 != 0 the three
 * gradients are written as fp32 so that per-block contributions can be summed without bf16 rounding. */
DF_API int df_attn_delta_bf16(const void *out, const void *d_out, float *delta, uint32_t batch, uint32_t n_heads,
                       uint32_t seq_len, uint32_t d_head, void *stream);
DF_API int df_attn_backward_block_bf16(const void *q, const void *k, const void *v, const void *d_out, const float *lse,
                                const float *delta, void *d_q, void *d_k, void *d_v, uint32_t batch,
                                uint32_t n_heads, uint32_t seq_q, uint32_t seq_k, uint32_t d_head, float scale,
                                uint32_t causal, int64_t causal_shift, uint32_t out_fp32, void *stream);

/* delta[b,h,i] = sum_d dO[b,i,h,d] * O[b,i,h,d]: the row-sum pre-pass of the backward. */
DF_API int df_attn_delta(const float *out, const float *d_out, float *delta, uint32_t batch,
                  uint32_t n_heads, uint32_t seq_len, uint32_t d_head, void *stream);

/* Backward from saved out and lse. `delta` is caller scratch [B,H,S] floats, overwritten.
 * Extends launch_fused_mha_backward (attention_fused.cu:518-532): no S*S scratch. */
DF_API int df_attn_backward(const float *q, const float *k, const float *v, const float *out,
                     const float *d_out, const float *lse, float *d_q, float *d_k, float *d_v,
                     float *delta, uint32_t batch, uint32_t n_heads, uint32_t seq_len,
                     uint32_t d_head, float scale, uint32_t causal, void *stream);

/* Optional one-time set-up for the calling thread on the current device (no counterpart in the
 * reference). The library creates CUDA objects in exactly one situation: df_attn_backward_block runs
 * its two independent kernels on two streams, and the second stream with its fork/join events
 * belongs to the calling thread (so concurrent callers never share them). They are created here, or
 * else by that thread's first df_attn_backward_block on the device; call this first when that first
 * call would fall inside a stream capture or a no-allocation region. Every other entry point
 * creates nothing, ever. */
DF_API int df_attn_init(void);

/* df_attn_backward plus the device time of its two kernels, for benchmarks: launches the dQ (+ delta)
 * kernel four times back to back, then the dK/dV kernel four times (an event pair around a single
 * launch would add several microseconds to a 70-microsecond kernel), with events before, between
 * and after the two groups; synchronises the stream and returns the two durations per launch in
 * milliseconds (0 when the SIMT path ran, which runs once). Creates and destroys three events per
 * call: a measurement aid, not part of the allocation-free contract. Results are the same as
 * df_attn_backward's. No counterpart in the reference. */
DF_API int df_attn_backward_profile(const float *q, const float *k, const float *v, const float *out,
                             const float *d_out, const float *lse, float *d_q, float *d_k, float *d_v,
                             float *delta, uint32_t batch, uint32_t n_heads, uint32_t seq_len,
                             uint32_t d_head, float scale, uint32_t causal, void *stream, float *ms_dq,
                             float *ms_dkdv);

/* Backward for callers that cannot hand over scratch memory. It has no counterpart in the
 * reference (whose backward always takes a caller-allocated `probabilities` buffer); it exists
 * for hosts that may not allocate at call time and have no spare buffer to lend: an engine that
 * carved up all of its device memory into fixed tensors when it was constructed, or a plugin
 * host that forbids allocator calls from inside an operator. Same result as df_attn_backward,
 * but the delta row sums live in an array compiled into the library instead of a `delta`
 * argument, and the call performs no cudaMalloc / cudaFree / allocating library routine.
 *   - Limit: batch * n_heads * seq_len <= DF_STATIC_SCRATCH_MAX_ROWS (8 MiB of floats that every
 *     GPU which loads the library holds until the process exits). Larger problems are refused
 *     with DF_ERR_STATIC_SCRATCH and nothing is launched.
 *   - The first call on each device looks up the array's device address (once per device, with
 *     that device current). Make that first call outside any stream capture.
 *   - All calls share the one array and it keeps whatever the previous call left in it. Nothing
 *     in it needs to start at zero: each call overwrites the rows it is about to read. Two calls
 *     whose kernels can overlap on the GPU (different streams, different threads) race on it;
 *     serialise them, or use df_attn_backward with separate delta buffers. */
#define DF_STATIC_SCRATCH_MAX_ROWS 2097152u
DF_API int df_attn_backward_static_scratch(const float *q, const float *k, const float *v, const float *out,
                                    const float *d_out, const float *lse, float *d_q, float *d_k,
                                    float *d_v, uint32_t batch, uint32_t n_heads, uint32_t seq_len,
                                    uint32_t d_head, float scale, uint32_t causal, void *stream);

/* Block form of the backward for ring steps: adds nothing to memory beyond its outputs.
 * d_q [B,Sq,H*D] and d_k,d_v [B,Sk,H*D] are overwritten with this block's contribution;
 * lse and delta [B,H,Sq] are the FINAL (merged) row statistics. */
DF_API int df_attn_backward_block(const float *q, const float *k, const float *v, const float *d_out,
                           const float *lse, const float *delta, float *d_q, float *d_k,
                           float *d_v, uint32_t batch, uint32_t n_heads, uint32_t seq_q,
                           uint32_t seq_k, uint32_t d_head, float scale, uint32_t causal,
                           int64_t causal_shift, void *stream);

/* Merge two partial results over disjoint key sets, in place into (o_a, lse_a):
 * lse = logaddexp(lse_a, lse_b); O = e^(lse_a-lse) O_a + e^(lse_b-lse) O_b. Same rescale as
 * the split-K decode reduction, attention_fused.cu:714-760. */
DF_API int df_attn_merge_partials(float *o_a, float *lse_a, const float *o_b, const float *lse_b,
                           uint32_t batch, uint32_t n_heads, uint32_t seq_len, uint32_t d_head,
                           void *stream);

/* Accumulate: dst += src over n floats (ring backward: summing per-block dQ / dK / dV). */
DF_API int df_attn_accumulate(float *dst, const float *src, uint64_t n, void *stream);

/* ---- the projections on either side of the attention op ----
 * out[rows, out_features] = x[rows, in_features] W[out_features, in_features]^T + bias[out_features] (+ residual),
 * row-major fp32 like the reference's DeviceTensor::linear_into (darkforest-cuda/src/lib.rs:1138-1201: cublasSgemm,
 * then launch_add_bias, darkforest-cuda/kernels/elementwise.cu:230-249).
 *   df_linear_qkv_forward  replaces the three Q/K/V projections of a layer, i.e. three linear_into calls = three
 *       GEMMs and three bias passes (darkforest-core/src/engine/static_gpt2.rs:1324-1326), by one launch that
 *       writes q, k, v [rows, out_features] in the [S, H*D] layout the attention entry points read. The three
 *       biases are all given or all NULL.
 *   df_linear_forward      one projection with optional bias and optional residual[rows, out_features] added in
 *       the epilogue: the output projection, its bias pass and the first residual add (static_gpt2.rs:1339-1341).
 * One persistent tcgen05 kernel: x and W rounded to TF32 in flight, fp32 accumulation, bias/residual added in fp32
 * (the reference's cublasSgemm multiplies in full fp32; the difference is bounded like the attention op's:
 * about 1e-3 of the output's scale at in_features = 768). in_features and out_features must be multiples of 4
 * and all pointers 16-byte aligned, else DF_ERR_UNSUPPORTED (there is no other path); out must not alias x or residual. */
DF_API int df_linear_qkv_forward(const float *x, const float *wq, const float *wk, const float *wv, const float *bq,
                          const float *bk, const float *bv, float *q, float *k, float *v, uint32_t rows,
                          uint32_t in_features, uint32_t out_features, void *stream);
DF_API int df_linear_forward(const float *x, const float *w, const float *bias, const float *residual, float *out,
                      uint32_t rows, uint32_t in_features, uint32_t out_features, void *stream);
/* The MLP's first projection with its activation in the epilogue: pre_activation = x w^T + bias and
 * out = gelu(pre_activation) (tanh form, the arithmetic of df_gelu_forward) from one pass over the accumulators.
 * Replaces linear_into + gelu_into of darkforest-core/src/engine/static_gpt2.rs:1353-1355 (cublasSgemm, bias pass,
 * launch_gelu: the [rows, out_features] activation is written once and never re-read). pre_activation is what
 * df_gelu_backward needs (la.mlp_h); NULL skips it (inference). Same shape and alignment rules as df_linear_forward;
 * out must not alias x or pre_activation. */
DF_API int df_linear_gelu_forward(const float *x, const float *w, const float *bias, float *pre_activation, float *out,
                           uint32_t rows, uint32_t in_features, uint32_t out_features, void *stream);

/* ---- the row-wise and elementwise kernels of the training step around attention ----
 * Legacy symbols (legacy stream, no status), same arguments and arithmetic as the reference's:
 *   launch_layernorm           replaces darkforest-cuda/kernels/layernorm.cu:97-108 (kernels.rs:603-640): per row of
 *       x[rows, cols]: mean, rstd = 1 / sqrt(var + 1e-5) (biased variance), out = (x - mean) * rstd * gamma + beta;
 *       gamma, beta, means, rstds may each be NULL (1, 0, not stored).
 *   launch_layernorm_backward  replaces layernorm.cu:187-200: grad_x = rstd / cols * (cols * ds - sum(ds) - xhat * sum(ds * xhat))
 *       with ds = grad_out * gamma; grad_gamma += sum over rows of grad_out * xhat and grad_beta += sum over rows of
 *       grad_out are ADDED to what the buffers hold (the caller zeroes them, as the reference's callers do); either may be NULL.
 *   launch_gelu / launch_gelu_backward  replace kernels/elementwise.cu:195-199, 217-224 (tanh form of GELU).
 *   launch_adamw_update        replaces kernels/matmul.cu:341-363: m = b1 m + (1 - b1) g; v = b2 v + (1 - b2) g^2;
 *       p = p (1 - lr wd) - lr (m / bias_correction1) / (sqrt(v / bias_correction2) + eps).
 * The static step calls them per layer and per parameter tensor (darkforest-core/src/engine/static_gpt2.rs:1314-1364,
 * 1426-1500, 1651-1700). The df_* forms add a status and a stream and take 64-bit element counts. The LayerNorm
 * kernels read each activation once per pass where the reference reads it two to three times, and issue one global
 * atomic per column and thread block for grad_gamma / grad_beta instead of two per element (the sums are therefore
 * still order-dependent in the last bits, like the reference's).
 * df_adamw_update_multi updates every tensor of a table in ONE launch (the reference launches once per tensor:
 * 196 launches for a 12-layer GPT-2 small). The caller fills `parameter`, `first_moment`, `second_moment`, `gradient`, `n` of each
 * entry on the host, calls df_adamw_plan (host only: fills `first_chunk`, returns the number of work units), copies the
 * table into device memory it owns and passes that pointer with the returned count. No counterpart in the reference. */
typedef struct df_adamw_tensor {
  float *parameter;
  float *first_moment;
  float *second_moment;
  const float *gradient;
  uint64_t n;           /* elements */
  uint64_t first_chunk; /* filled by df_adamw_plan */
} df_adamw_tensor_t;
DF_API void launch_layernorm(const float *x, const float *gamma, const float *beta, float *out, float *means, float *rstds,
                      uint32_t batch, uint32_t features);
DF_API void launch_layernorm_backward(const float *grad_out, const float *x, const float *gamma, const float *means,
                               const float *rstds, float *grad_x, float *grad_gamma, float *grad_beta, uint32_t batch,
                               uint32_t features);
DF_API void launch_gelu(const float *x, float *out, uint32_t n);
DF_API void launch_gelu_backward(const float *grad_out, const float *x, float *grad_x, uint32_t n);
DF_API void launch_adamw_update(float *parameter, float *first_moment, float *second_moment, const float *gradient, uint32_t n,
                         float lr, float beta1, float beta2, float eps, float weight_decay, float bias_correction1,
                         float bias_correction2);
DF_API int df_layernorm_forward(const float *x, const float *gamma, const float *beta, float *out, float *means, float *rstds,
                         uint32_t rows, uint32_t cols, void *stream);
DF_API int df_layernorm_backward(const float *grad_out, const float *x, const float *gamma, const float *means,
                          const float *rstds, float *grad_x, float *grad_gamma, float *grad_beta, uint32_t rows,
                          uint32_t cols, void *stream);
DF_API int df_gelu_forward(const float *x, float *out, uint64_t n, void *stream);
DF_API int df_gelu_backward(const float *grad_out, const float *x, float *grad_x, uint64_t n, void *stream);
DF_API int df_adamw_update(float *parameter, float *first_moment, float *second_moment, const float *gradient, uint64_t n,
                    float lr, float beta1, float beta2, float eps, float weight_decay, float bias_correction1,
                    float bias_correction2, void *stream);
DF_API uint64_t df_adamw_plan(df_adamw_tensor_t *tensors_host, uint32_t n_tensors);
DF_API int df_adamw_update_multi(const df_adamw_tensor_t *tensors_device, uint32_t n_tensors, uint64_t total_chunks, float lr,
                          float beta1, float beta2, float eps, float weight_decay, float bias_correction1,
                          float bias_correction2, void *stream);

/* ---- the loss head's fused softmax + cross-entropy over one chunk of logits (legacy symbols, legacy stream) ----
 *   launch_fused_chunked_logit_ce  replaces darkforest-cuda/kernels/softmax.cu:325-410 (kernels.rs:531-566): logits
 *       [chunk_rows, cols] become probabilities in place, grad_logits = (p - onehot(target)) / total_rows,
 *       *loss += sum over the rows of -log(max(p[target], 1e-12)) / total_rows. targets[chunk_rows] are u32 token ids.
 *   launch_chunked_ce_eval         replaces softmax.cu:415-480 (kernels.rs:568-600): loss only, logits untouched.
 * The static step calls them once per 512-row chunk (darkforest-core/src/engine/static_gpt2.rs:1386-1418). Each row
 * is read from global memory once (it stays in shared memory between the passes; the reference reads it three times).
 * df_chunked_logit_ce is both with a status and a stream: grad_logits NULL selects the eval form. */
DF_API void launch_fused_chunked_logit_ce(float *logits, const uint32_t *targets, float *grad_logits, float *loss,
                                   uint32_t chunk_rows, uint32_t cols, uint32_t total_rows);
DF_API void launch_chunked_ce_eval(float *logits, const uint32_t *targets, float *loss, uint32_t chunk_rows, uint32_t cols,
                            uint32_t total_rows);
DF_API int df_chunked_logit_ce(float *logits, const uint32_t *targets, float *grad_logits, float *loss, uint32_t chunk_rows,
                        uint32_t cols, uint32_t total_rows, void *stream);

/* ---- variant selection and status ---- */
#define DF_VARIANT_AUTO 0     /* tensor-core kernel where the shape allows, SIMT otherwise */
#define DF_VARIANT_SIMT 1     /* force the shape-generic SIMT kernels                      */
#define DF_VARIANT_TENSOR 2   /* force the tcgen05 kernels; unsupported shapes return DF_ERR_UNSUPPORTED */
DF_API int df_attn_set_variant(int variant);  /* per calling thread; returns the previous value */

/* Process-wide tuning options (no counterpart in the reference). Each option starts from the
 * environment variable named beside it, read ONCE when the library first looks an option up; after
 * that only df_attn_set_option changes it (returns the previous value, -1 for an unknown option).
 * None of them changes results beyond rounding order; no launcher reads the environment. */
#define DF_OPT_FWD_PERSIST 0     /* DF_ATTN_FWD_PERSIST: persistent TF32 forward 0 never, 1 up to S = 2048 (default), 2 always */
#define DF_OPT_FUSE_DELTA 1      /* DF_ATTN_FUSE_DELTA: 1 (default) the dQ kernel forms delta itself, 0 separate pre-pass    */
#define DF_OPT_BWD_OVERLAP 2     /* DF_ATTN_BWD_OVERLAP: 1 (default) block backward runs dQ on the thread's side stream      */
#define DF_OPT_SCHED_TABLE 3     /* DF_ATTN_SCHED_TABLE: 1 (default) explicit work lists for the persistent forward          */
#define DF_OPT_DISABLE_TENSOR 4  /* DF_ATTN_DISABLE_TENSOR: 1 = SIMT kernels only, 2 = SIMT backward only (default 0)        */
#define DF_OPT_PDL 5             /* DF_ATTN_PDL: 1 = launch the TF32 kernels with programmatic stream serialization; default 0:
                                    measured slower on B200 (fwd+bwd step 0.243 vs 0.221 ms) */
#define DF_OPT_CE_VARIANT 6      /* DF_CE_VARIANT: loss-head training kernel 0 = automatic, 1 = row resident in shared memory,
                                    2 = two passes, the second out of L2 */
#define DF_OPT_LN_STAGED 7       /* DF_LN_STAGED: 1 (default) the LayerNorm backward stages its rows in shared memory with bulk
                                    copies when there are enough rows to fill the machine, 0 = rows in registers only          */
#define DF_OPT_COUNT 8
DF_API int df_attn_set_option(int option, int value);
DF_API int df_attn_get_option(int option);

/* 1 if the tensor-core path would be taken for this forward problem under AUTO. */
DF_API int df_attn_forward_uses_tensor_cores(const void *q, const void *k, const void *v, const void *out,
                                      uint32_t n_heads, uint32_t seq_q, uint32_t seq_k,
                                      uint32_t d_head);

DF_API int df_attn_last_status(void);              /* sticky status of the calling thread; clears it */
DF_API const char *df_attn_status_string(int status);
/* Failure-path self-test: launches one small kernel that waits, with the library's bounded wait, on a
 * barrier that nothing will ever signal, with a budget of `budget_ms` milliseconds (1..2000). The wait
 * gives up, the kernel exits normally and raises the device status bit, so the next df_sync_status()
 * returns DF_ERR_DEVICE_TIMEOUT (and clears it) while the context stays usable. The reference has no
 * counterpart: its kernels trap on bad input (attention_fused.cu:56-58) and its sync aborts. */
DF_API int df_attn_selftest_wait_expiry(uint32_t budget_ms, void *stream);

/* Checked builds (make EXTRA=-DDF_BOUNDS_CHECK; no counterpart in the reference, which runs unchecked): the
 * SIMT kernels range-check every global-memory index; an index outside its tensor sets a bit in the device status word
 * and is replaced by 0, so nothing outside the tensor is touched and the context stays usable, and df_sync_status
 * returns DF_ERR_DEVICE_BOUNDS once. This call makes one thread ask the checker for an out-of-range element, which is
 * how a test sees the path work without a bad access. In a normal build it returns DF_ERR_UNSUPPORTED. */
DF_API int df_attn_selftest_bounds_check(void *stream);

/* cudaDeviceSynchronize + device status word; never aborts. */
DF_API int df_sync_status(void);
/* Number of kernels this library launched from the calling thread since the last reset. */
DF_API uint64_t df_attn_launch_count(int reset);
DF_API const char *df_attn_build_info(void);

#ifdef __cplusplus
}
#endif
#endif /* DARKFOREST_KERNELS_H */
