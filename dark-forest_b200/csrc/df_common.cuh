// df_common.cuh — shared declarations of the attention library (host + device).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/darkforest_kernels.h"

// Optional NVTX ranges around the entry points (make NVTX=1 adds -DDF_NVTX; the header-only NVTX v3 needs no
// library): a profiler timeline then shows which public call a kernel belongs to. Compiled out by default.
#ifdef DF_NVTX
#include <nvtx3/nvToolsExt.h>
namespace df {
struct NvtxRange {
  explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};
}  // namespace df
#define DF_RANGE(name) ::df::NvtxRange df_nvtx_range_(name)
#else
#define DF_RANGE(name) \
  do {                 \
  } while (0)
#endif

namespace df {

// One attention problem (or one block of a ring-partitioned problem).
// Layout: q-side tensors [B][Sq][H*D], k-side tensors [B][Sk][H*D], row statistics [B][H][Sq].
struct AttnParams {
  const float *q = nullptr, *k = nullptr, *v = nullptr;
  const float *o_in = nullptr;    // saved forward output (backward / delta)
  const float *d_out = nullptr;   // dO
  const float *lse_in = nullptr;  // saved logsumexp (backward)
  const float *delta_in = nullptr;
  float *out = nullptr, *lse = nullptr, *delta = nullptr;
  float *d_q = nullptr, *d_k = nullptr, *d_v = nullptr;
  uint32_t B = 1, H = 1, Sq = 0, Sk = 0, D = 0;
  int out_f32 = 0;  // bf16 variant only: results (out, or d_q/d_k/d_v) are written as fp32 instead of bf16
  int bf16 = 0;  // 1: q, k, v, out (and d_out, d_q, d_k, d_v, o_in) point at bf16 elements; lse/delta stay fp32
  float scale = 1.0f;
  int causal = 0;
  long long shift = 0;  // key j visible to query i iff !causal or j <= i + shift
  unsigned int *status = nullptr;  // device status word (checked builds of the SIMT kernels; set by their launchers)
};

// Sticky per-thread status and launch counter (defined in attn_api.cu).
void note_status(int status);
void note_launch(int n = 1);
int check_cuda(cudaError_t e);  // maps to DF_ERR_CUDA and records it

// Device status word of the current device: kernels OR a bit in when a bounded wait gives up;
// df_sync_status reads and clears it. The pointer is resolved once per device, without allocating.
unsigned int *device_status_ptr();
// Process-wide tuning options (include/darkforest_kernels.h: DF_OPT_*). Each starts from its
// environment variable, read once when the first option is looked up, and can be changed at run time
// with df_attn_set_option; no launcher calls getenv.
int option(int which);
constexpr unsigned int DEV_STATUS_WAIT_EXPIRED = 1u;
constexpr unsigned int DEV_STATUS_BOUNDS = 2u;

// Optional checked build (make EXTRA=-DDF_BOUNDS_CHECK): every global-memory index of the SIMT kernels goes through
// DF_IDX(i, n, status): an index outside [0, n) ORs DEV_STATUS_BOUNDS into the device status word and is replaced by 0,
// so the access itself stays inside the tensor and the context stays usable; df_sync_status then returns
// DF_ERR_DEVICE_BOUNDS. In the normal build the macro is the index itself. (The tensor-core kernels move their
// tiles with TMA, whose tensor maps bound every copy in hardware.)
#ifdef DF_BOUNDS_CHECK
#ifdef __CUDACC__
__device__ __forceinline__ size_t df_checked_index(size_t i, size_t n, unsigned int *status) {
  if (i < n) return i;
  if (status) atomicOr(status, DEV_STATUS_BOUNDS);
  return 0;
}
#endif
#define DF_IDX(i, n, status) df_checked_index((size_t)(i), (size_t)(n), (status))
#else
#define DF_IDX(i, n, status) (i)
#endif

// ---- SIMT kernels, any shape (attn_generic.cu) ----
int generic_forward(const AttnParams &p, cudaStream_t s);            // out/lse and/or delta (stats mode)
int generic_backward_dkdv(const AttnParams &p, cudaStream_t s);      // needs lse_in, delta_in
int generic_backward_dq(const AttnParams &p, cudaStream_t s);
int delta_prepass(const AttnParams &p, cudaStream_t s);              // delta = rowsum(dO * O)
int merge_partials(float *o_a, float *lse_a, const float *o_b, const float *lse_b, uint32_t B,
                   uint32_t H, uint32_t S, uint32_t D, cudaStream_t s);
int accumulate(float *dst, const float *src, uint64_t n, cudaStream_t s);

// ---- tcgen05 kernels (attn_fwd_sm100.cu / attn_bwd_sm100.cu) ----
bool tensor_forward_supported(const AttnParams &p);
int tensor_forward(const AttnParams &p, cudaStream_t s);
bool tensor_backward_supported(const AttnParams &p);
int tensor_backward(const AttnParams &p, cudaStream_t s);
// Creates, for the calling thread and the current device, what the block backward would otherwise
// create on its first call: the side stream and its two events; also sets the kernel attributes.
int tensor_backward_init();
// Profiling hook of the calling thread: with a non-null array of three events the next backward
// launches record ev[0] / ev[1] / ev[2] before, between and after the dQ and dK/dV kernels on the
// caller's stream (and run them strictly one after the other).
void tensor_backward_set_profile_events(cudaEvent_t *three_events);
constexpr int kProfileReps = 4;  // launches of each kernel between the events of a profiled backward
// Static schedule of the persistent kernels: work items are numbered heaviest first and dealt to the
// `grid` CTAs in rounds, odd rounds in reverse CTA order ("snake"), which on the causal triangle
// balances as well as a greedy longest-first assignment and needs no counter that concurrent
// launches could share. Returns the item of CTA `cta` in round `r`, or -1 when its list is exhausted.
__host__ __device__ inline long long snake_item(int r, int grid, int cta, long long n_items) {
  const long long idx = (long long)r * grid + ((r & 1) ? (grid - 1 - cta) : cta);
  return idx < n_items ? idx : -1;
}

// Optional explicit work lists for the persistent kernels. The snake formula is as good as greedy
// longest-first, but with few heavy items per CTA (one long sequence, a dozen heads) neither is
// close to the average load: at S = 8192, B*H = 12 the heaviest CTA carries 96 steps against an
// average of 85.6. For up to kSchedMaxItems items the forward launcher therefore computes a MULTIFIT
// assignment on the host (first-fit decreasing under a binary-searched capacity, cached per shape)
// and passes it to the kernel as a parameter: CTA c runs items[off[c] .. off[c+1]) in that order
// (measured on B200, B=1, H=12: forward at S = 8192 351 -> 381 TFLOP/s, S = 16384 404 -> 410). The
// backward kernels keep the snake order: the same tables made them slower (S = 4096: 0.34 -> 0.38-0.43
// ms, S = 8192: 0.96 -> 1.03-1.05 ms, whatever weight the change of tile was given).
constexpr int kSchedMaxItems = 2048;
constexpr int kSchedMaxCtas = 160;
struct SchedTable {
  uint32_t used;                       // 0: no table, the kernel uses snake_item
  uint16_t off[kSchedMaxCtas + 2];
  uint16_t items[kSchedMaxItems];
};
__host__ __device__ inline long long sched_item(const SchedTable &t, int r, int grid, int cta, long long n_items) {
  if (t.used) {
    const int i = (int)t.off[cta] + r;
    return i < (int)t.off[cta + 1] ? (long long)t.items[i] : -1;
  }
  return snake_item(r, grid, cta, n_items);
}
// Fills `out` for `n_items` items of the given weights (any order) on `grid` CTAs; out->used = 0 when
// the table does not apply (too many items, one round at most, or no better than the snake order).
// `key` identifies the shape for the per-process cache (attn_sched.cu).
struct SchedKey {
  int kind;  // 0 forward pairs (the only user so far)
  uint32_t bh, sq, sk;
  int causal;
  long long shift;
  int grid;
};
void schedule_for(const SchedKey &key, int n_items, uint32_t (*weight)(const void *ctx, int item), const void *ctx,
                  SchedTable *out);

// one-token decode over a contiguous or paged KV cache (attn_decode.cu)
int decode_dispatch(const float *q, const void *k, const void *v, const int32_t *block_table, float *out,
                    float *partial_m, float *partial_l, float *partial_o, uint32_t max_chunks, uint32_t H,
                    uint32_t T, uint32_t D, float scale, uint32_t page_size, bool kv_bf16, cudaStream_t s);
// persistent TF32 forward for whole sequences with head dimension 64 (attn_fwd_persist_sm100.cu)
bool tensor_forward_persistent_supported(const AttnParams &p);
int tensor_forward_persistent(const AttnParams &p, cudaStream_t s);

// ---- projections around the attention op (linear_sm100.cu): out_j = X W_j^T + b_j (+ residual), j < n_mats <= 3 ----
bool tensor_linear_supported(const float *x, const float *const *w, const float *const *bias, float *const *out,
                             const float *residual, int n_mats, uint32_t M, uint32_t K, uint32_t N);
int tensor_linear(const float *x, const float *const *w, const float *const *bias, float *const *out, const float *residual,
                  float *gelu_out,
                  int n_mats, uint32_t M, uint32_t K, uint32_t N, cudaStream_t s);

// tanh-form GELU of the reference (kernels/elementwise.cu:180-215), shared by the elementwise kernels and the projection
// kernel's epilogue so that the fused and the separate form give the same bits:
// gelu(v) = 0.5 v (1 + tanh u), u = sqrt(2/pi) (v + 0.044715 v^3); with s = 1 / (1 + exp(-2u)): tanh u = 2s - 1,
// so gelu = v s and gelu' = s + 2 v s (1 - s) u'.
#ifdef __CUDACC__
__device__ __forceinline__ float gelu_sigmoid(float v) {
  const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
  return __fdividef(1.0f, 1.0f + __expf(-2.0f * u));
}
__device__ __forceinline__ float gelu_value(float v) { return v * gelu_sigmoid(v); }
__device__ __forceinline__ float gelu_slope(float v) {
  const float s = gelu_sigmoid(v);
  const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * v * v);
  return s + 2.0f * v * s * (1.0f - s) * du;
}
#endif

// ---- LayerNorm, GELU, AdamW of the training step (step_kernels.cu) ----
int layernorm_forward(const float *x, const float *gamma, const float *beta, float *out, float *means, float *rstds,
                      uint32_t rows, uint32_t cols, cudaStream_t s);
int layernorm_backward(const float *grad_out, const float *x, const float *gamma, const float *means, const float *rstds,
                       float *grad_x, float *grad_gamma, float *grad_beta, uint32_t rows, uint32_t cols, cudaStream_t s);
int gelu_forward(const float *x, float *out, uint64_t n, cudaStream_t s);
int gelu_backward(const float *grad_out, const float *x, float *grad_x, uint64_t n, cudaStream_t s);
int adamw_update(float *p, float *m, float *v, const float *g, uint64_t n, float lr, float beta1, float beta2, float eps,
                 float weight_decay, float bc1, float bc2, cudaStream_t s);
uint64_t adamw_plan(df_adamw_tensor_t *tensors, uint32_t n_tensors);
int adamw_update_multi(const df_adamw_tensor_t *tensors_device, uint32_t n_tensors, uint64_t total_chunks, float lr, float beta1,
                       float beta2, float eps, float weight_decay, float bc1, float bc2, cudaStream_t s);
// ---- loss head: softmax + cross-entropy over one chunk of logits (loss_ce.cu); grad_logits == nullptr: eval form ----
int chunked_logit_ce(float *logits, const uint32_t *targets, float *grad_logits, float *loss, uint32_t chunk_rows, uint32_t cols,
                     uint32_t total_rows, cudaStream_t s);

// ---- bf16 variant of the backward (attn_bwd_bf16_sm100.cu) ----
bool tensor_backward_bf16_supported(const AttnParams &p);
int tensor_backward_bf16(const AttnParams &p, cudaStream_t s);
int delta_prepass_bf16(const AttnParams &p, cudaStream_t s);

}  // namespace df
