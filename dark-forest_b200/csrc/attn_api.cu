// attn_api.cu — the extern "C" boundary: argument validation, variant dispatch, status.
//
// The five legacy symbols keep the reference's names and signatures
// (darkforest-cuda/kernels/attention_fused.cu:223-226, 233-237, 361-366, 518-521 and
// darkforest-cuda/kernels/matmul.cu:21) so that darkforest-cuda/src/kernels.rs links unchanged.
// Nothing here allocates device memory; there is no CPU fallback: when a CUDA launch is not
// possible the call reports an error status.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "df_common.cuh"
#include "sm100_ptx.cuh"

namespace df {

namespace {
thread_local int t_status = DF_OK;
thread_local int t_variant = DF_VARIANT_AUTO;
thread_local uint64_t t_launches = 0;

__device__ unsigned int g_device_status_word = 0;
}  // namespace

void note_status(int status) {
  if (status != DF_OK && t_status == DF_OK) t_status = status;
}
void note_launch(int n) { t_launches += (uint64_t)n; }
int check_cuda(cudaError_t e) {
  if (e == cudaSuccess) return DF_OK;
  note_status(DF_ERR_CUDA);
  return DF_ERR_CUDA;
}

namespace {
std::atomic<int> g_options[DF_OPT_COUNT];
std::once_flag g_options_once;
void init_options() {
  auto rd = [](const char *name, int dflt) {
    const char *v = getenv(name);
    return v ? atoi(v) : dflt;
  };
  g_options[DF_OPT_FWD_PERSIST].store(rd("DF_ATTN_FWD_PERSIST", 1));
  g_options[DF_OPT_FUSE_DELTA].store(rd("DF_ATTN_FUSE_DELTA", 1));
  g_options[DF_OPT_BWD_OVERLAP].store(rd("DF_ATTN_BWD_OVERLAP", 1));
  g_options[DF_OPT_SCHED_TABLE].store(rd("DF_ATTN_SCHED_TABLE", 1));
  g_options[DF_OPT_DISABLE_TENSOR].store(rd("DF_ATTN_DISABLE_TENSOR", 0));
  g_options[DF_OPT_PDL].store(rd("DF_ATTN_PDL", 0));
  g_options[DF_OPT_CE_VARIANT].store(rd("DF_CE_VARIANT", 0));
  g_options[DF_OPT_LN_STAGED].store(rd("DF_LN_STAGED", 1));
}
}  // namespace

int option(int which) {
  std::call_once(g_options_once, init_options);
  return (which >= 0 && which < DF_OPT_COUNT) ? g_options[which].load(std::memory_order_relaxed) : 0;
}

unsigned int *device_status_ptr() {
  // One lookup per device; cudaGetSymbolAddress neither allocates nor synchronises.
  constexpr int kMaxDev = 64;
  static unsigned int *cache[kMaxDev] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  unsigned int *p = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void *addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_device_status_word) != cudaSuccess) return nullptr;
    p = static_cast<unsigned int *>(addr);
    __atomic_store_n(&cache[dev], p, __ATOMIC_RELEASE);
  }
  return p;
}

namespace {

bool size_ok(uint64_t B, uint64_t H, uint64_t S, uint64_t D) {
  // element counts must fit 2^62 so that byte offsets stay inside size_t
  const unsigned __int128 n = (unsigned __int128)B * H * S * D;
  return n < ((unsigned __int128)1 << 60);
}

int validate(uint32_t B, uint32_t H, uint32_t Sq, uint32_t Sk, uint32_t D) {
  if (D == 0 || D > 128) return DF_ERR_INVALID_ARG;  // darkforest-cuda/src/lib.rs:1981
  if (H == 0) return DF_ERR_INVALID_ARG;
  if (!size_ok(B, H, Sq > Sk ? Sq : Sk, D)) return DF_ERR_INVALID_ARG;
  if ((uint64_t)B * H > 0x7fffffffull) return DF_ERR_INVALID_ARG;
  return DF_OK;
}

int forward_dispatch(const AttnParams &p, cudaStream_t s) {
  if (p.B == 0 || p.Sq == 0) return DF_OK;
  if (t_variant == DF_VARIANT_SIMT) return generic_forward(p, s);
  const bool tensor_ok = p.out != nullptr && tensor_forward_supported(p);
  if (t_variant == DF_VARIANT_TENSOR) return tensor_ok ? tensor_forward(p, s) : DF_ERR_UNSUPPORTED;
  return tensor_ok ? tensor_forward(p, s) : generic_forward(p, s);
}

int backward_dispatch(const AttnParams &p, cudaStream_t s) {
  if (p.B == 0) return DF_OK;
  const bool tensor_ok = tensor_backward_supported(p);
  if (t_variant == DF_VARIANT_TENSOR && !tensor_ok) return DF_ERR_UNSUPPORTED;
  if (t_variant != DF_VARIANT_SIMT && tensor_ok) return tensor_backward(p, s);
  int st = generic_backward_dkdv(p, s);
  if (st != DF_OK) return st;
  return generic_backward_dq(p, s);
}

int finish(int st) {
  note_status(st);
  return st;
}

// Backward of a whole sequence from the saved output: p carries q, k, v, o_in, d_out, lse_in, the
// gradients and `delta`, a [B, H, S] buffer that holds rowsum(dO o O) afterwards. The tensor-core
// path computes those row sums inside its dQ kernel; every other path runs the pre-pass first.
int full_backward(AttnParams p, cudaStream_t s) {
  if (p.B == 0 || p.Sq == 0) return DF_OK;
  p.delta_in = nullptr;
  const bool aligned = (reinterpret_cast<uintptr_t>(p.o_in) & 15u) == 0;
  if (t_variant != DF_VARIANT_SIMT && aligned && option(DF_OPT_FUSE_DELTA) && tensor_backward_supported(p))
    return tensor_backward(p, s);
  int st = delta_prepass(p, s);
  if (st != DF_OK) return st;
  p.delta_in = p.delta;
  p.delta = nullptr;
  p.o_in = nullptr;
  return backward_dispatch(p, s);
}

// Legacy backward: the caller supplies only Q, K, V, dO and `scratch_floats` floats of scratch
// (H*2*S*S for the multi-head entry, S*S for the single-head one). O and the row statistics are
// recomputed into that scratch; when it is too small for O (tiny S), the statistics are
// computed without materialising O.
int legacy_backward(const float *q, const float *k, const float *v, const float *d_out, float *d_q,
                    float *d_k, float *d_v, float *scratch, uint64_t scratch_floats, uint32_t H,
                    uint32_t S, uint32_t D, float scale, uint32_t causal) {
  int st = validate(1, H, S, S, D);
  if (st != DF_OK) return st;
  if (S == 0) return DF_OK;
  if (!q || !k || !v || !d_out || !d_q || !d_k || !d_v) return DF_ERR_INVALID_ARG;
  cudaStream_t s = 0;
  const size_t n = (size_t)S * H * D;
  if (S == 1) {
    // one key: P = 1, dS = 0  =>  dQ = dK = 0, dV = dO
    if (check_cuda(cudaMemsetAsync(d_q, 0, n * sizeof(float), s)) != DF_OK) return DF_ERR_CUDA;
    if (check_cuda(cudaMemsetAsync(d_k, 0, n * sizeof(float), s)) != DF_OK) return DF_ERR_CUDA;
    return check_cuda(cudaMemcpyAsync(d_v, d_out, n * sizeof(float), cudaMemcpyDeviceToDevice, s));
  }
  if (!scratch) return DF_ERR_INVALID_ARG;
  const uint64_t stats = 2ull * H * S;
  if (scratch_floats < stats) return DF_ERR_WORKSPACE;
  AttnParams p;
  p.q = q; p.k = k; p.v = v; p.d_out = d_out;
  p.B = 1; p.H = H; p.Sq = S; p.Sk = S; p.D = D;
  p.scale = scale; p.causal = causal != 0; p.shift = 0;
  if (scratch_floats >= (uint64_t)n + stats) {
    float *o = scratch, *lse = scratch + n, *delta = lse + (size_t)H * S;
    p.out = o; p.lse = lse;
    st = forward_dispatch(p, s);
    if (st != DF_OK) return st;
    p.out = nullptr; p.lse = nullptr;
    p.o_in = o; p.delta = delta; p.lse_in = lse;
    p.d_q = d_q; p.d_k = d_k; p.d_v = d_v;
    return full_backward(p, s);
  } else {
    float *lse = scratch, *delta = scratch + (size_t)H * S;
    p.out = nullptr; p.lse = lse; p.delta = delta;
    st = generic_forward(p, s);
    if (st != DF_OK) return st;
    p.lse_in = lse; p.delta_in = delta;
  }
  p.out = nullptr; p.lse = nullptr; p.delta = nullptr;
  p.d_q = d_q; p.d_k = d_k; p.d_v = d_v;
  return backward_dispatch(p, s);
}

// One warp waits on an mbarrier that is never signalled; the bounded wait runs out after budget_ns.
__global__ void k_selftest_wait_expiry(unsigned long long budget_ns, unsigned int *status) {
  __shared__ uint64_t bar_storage;
  __shared__ uint32_t abort_word;
  const uint32_t bar = ptx::smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1);
    abort_word = 0;
    ptx::mbar_init_fence();
  }
  __syncthreads();
  const bool completed = ptx::mbar_wait_budget(bar, 0, &abort_word, budget_ns);
  __syncthreads();
  if (threadIdx.x == 0 && !completed && status) atomicOr(status, DEV_STATUS_WAIT_EXPIRED);
}

}  // namespace
}  // namespace df

using namespace df;

extern "C" {

int df_attn_forward_block(const float *q, const float *k, const float *v, float *out, float *lse,
                          uint32_t batch, uint32_t n_heads, uint32_t seq_q, uint32_t seq_k,
                          uint32_t d_head, float scale, uint32_t causal, int64_t causal_shift,
                          void *stream) {
  DF_RANGE("df_attn_forward_block");
  int st = validate(batch, n_heads, seq_q, seq_k, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || seq_q == 0) return DF_OK;
  if (!q || !out || (seq_k > 0 && (!k || !v))) return finish(DF_ERR_INVALID_ARG);
  AttnParams p;
  p.q = q; p.k = k; p.v = v; p.out = out; p.lse = lse;
  p.B = batch; p.H = n_heads; p.Sq = seq_q; p.Sk = seq_k; p.D = d_head;
  p.scale = scale; p.causal = causal != 0; p.shift = causal_shift;
  return finish(forward_dispatch(p, static_cast<cudaStream_t>(stream)));
}

int df_attn_forward_bf16(const void *q, const void *k, const void *v, void *out, float *lse,
                         uint32_t batch, uint32_t n_heads, uint32_t seq_q, uint32_t seq_k,
                         uint32_t d_head, float scale, uint32_t causal, int64_t causal_shift,
                         uint32_t out_fp32, void *stream) {
  DF_RANGE("df_attn_forward_bf16");
  int st = validate(batch, n_heads, seq_q, seq_k, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || seq_q == 0) return DF_OK;
  if (!q || !out || (seq_k > 0 && (!k || !v))) return finish(DF_ERR_INVALID_ARG);
  AttnParams p;
  p.q = static_cast<const float *>(q); p.k = static_cast<const float *>(k); p.v = static_cast<const float *>(v);
  p.out = static_cast<float *>(out); p.lse = lse;
  p.B = batch; p.H = n_heads; p.Sq = seq_q; p.Sk = seq_k; p.D = d_head;
  p.scale = scale; p.causal = causal != 0; p.shift = causal_shift;
  p.bf16 = 1; p.out_f32 = out_fp32 != 0;
  if (!tensor_forward_supported(p)) return finish(DF_ERR_UNSUPPORTED);  // no SIMT path for bf16
  return finish(tensor_forward(p, static_cast<cudaStream_t>(stream)));
}

int df_attn_delta_bf16(const void *out, const void *d_out, float *delta, uint32_t batch, uint32_t n_heads,
                       uint32_t seq_len, uint32_t d_head, void *stream) {
  int st = validate(batch, n_heads, seq_len, seq_len, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || seq_len == 0) return DF_OK;
  if (!out || !d_out || !delta) return finish(DF_ERR_INVALID_ARG);
  AttnParams p;
  p.o_in = static_cast<const float *>(out); p.d_out = static_cast<const float *>(d_out); p.delta = delta;
  p.B = batch; p.H = n_heads; p.Sq = seq_len; p.Sk = seq_len; p.D = d_head; p.bf16 = 1;
  return finish(delta_prepass_bf16(p, static_cast<cudaStream_t>(stream)));
}

int df_attn_backward_block_bf16(const void *q, const void *k, const void *v, const void *d_out, const float *lse,
                                const float *delta, void *d_q, void *d_k, void *d_v, uint32_t batch,
                                uint32_t n_heads, uint32_t seq_q, uint32_t seq_k, uint32_t d_head, float scale,
                                uint32_t causal, int64_t causal_shift, uint32_t out_fp32, void *stream) {
  DF_RANGE("df_attn_backward_block_bf16");
  int st = validate(batch, n_heads, seq_q, seq_k, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || (seq_q == 0 && seq_k == 0)) return DF_OK;
  if (!q || !k || !v || !d_out || !lse || !delta || !d_q || !d_k || !d_v) return finish(DF_ERR_INVALID_ARG);
  AttnParams p;
  p.q = static_cast<const float *>(q); p.k = static_cast<const float *>(k); p.v = static_cast<const float *>(v);
  p.d_out = static_cast<const float *>(d_out);
  p.d_q = static_cast<float *>(d_q); p.d_k = static_cast<float *>(d_k); p.d_v = static_cast<float *>(d_v);
  p.lse_in = lse; p.delta_in = delta;
  p.B = batch; p.H = n_heads; p.Sq = seq_q; p.Sk = seq_k; p.D = d_head;
  p.scale = scale; p.causal = causal != 0; p.shift = causal_shift;
  p.bf16 = 1; p.out_f32 = out_fp32 != 0;
  if (!tensor_backward_bf16_supported(p)) return finish(DF_ERR_UNSUPPORTED);
  return finish(tensor_backward_bf16(p, static_cast<cudaStream_t>(stream)));
}

int df_attn_backward_bf16(const void *q, const void *k, const void *v, const void *out, const void *d_out,
                          const float *lse, void *d_q, void *d_k, void *d_v, float *delta, uint32_t batch,
                          uint32_t n_heads, uint32_t seq_len, uint32_t d_head, float scale, uint32_t causal,
                          void *stream) {
  int st = df_attn_delta_bf16(out, d_out, delta, batch, n_heads, seq_len, d_head, stream);
  if (st != DF_OK) return st;
  return df_attn_backward_block_bf16(q, k, v, d_out, lse, delta, d_q, d_k, d_v, batch, n_heads, seq_len, seq_len, d_head,
                                     scale, causal, 0, 0, stream);
}

int df_attn_forward(const float *q, const float *k, const float *v, float *out, float *lse,
                    uint32_t batch, uint32_t n_heads, uint32_t seq_len, uint32_t d_head,
                    float scale, uint32_t causal, void *stream) {
  return df_attn_forward_block(q, k, v, out, lse, batch, n_heads, seq_len, seq_len, d_head, scale,
                               causal, 0, stream);
}

int df_attn_delta(const float *out, const float *d_out, float *delta, uint32_t batch,
                  uint32_t n_heads, uint32_t seq_len, uint32_t d_head, void *stream) {
  DF_RANGE("df_attn_delta");
  int st = validate(batch, n_heads, seq_len, seq_len, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || seq_len == 0) return DF_OK;
  if (!out || !d_out || !delta) return finish(DF_ERR_INVALID_ARG);
  AttnParams p;
  p.o_in = out; p.d_out = d_out; p.delta = delta;
  p.B = batch; p.H = n_heads; p.Sq = seq_len; p.Sk = seq_len; p.D = d_head;
  return finish(delta_prepass(p, static_cast<cudaStream_t>(stream)));
}

int df_attn_backward_block(const float *q, const float *k, const float *v, const float *d_out,
                           const float *lse, const float *delta, float *d_q, float *d_k,
                           float *d_v, uint32_t batch, uint32_t n_heads, uint32_t seq_q,
                           uint32_t seq_k, uint32_t d_head, float scale, uint32_t causal,
                           int64_t causal_shift, void *stream) {
  DF_RANGE("df_attn_backward_block");
  int st = validate(batch, n_heads, seq_q, seq_k, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || (seq_q == 0 && seq_k == 0)) return DF_OK;
  if (!q || !k || !v || !d_out || !lse || !delta || !d_q || !d_k || !d_v)
    return finish(DF_ERR_INVALID_ARG);
  AttnParams p;
  p.q = q; p.k = k; p.v = v; p.d_out = d_out; p.lse_in = lse; p.delta_in = delta;
  p.d_q = d_q; p.d_k = d_k; p.d_v = d_v;
  p.B = batch; p.H = n_heads; p.Sq = seq_q; p.Sk = seq_k; p.D = d_head;
  p.scale = scale; p.causal = causal != 0; p.shift = causal_shift;
  return finish(backward_dispatch(p, static_cast<cudaStream_t>(stream)));
}

int df_attn_backward(const float *q, const float *k, const float *v, const float *out,
                     const float *d_out, const float *lse, float *d_q, float *d_k, float *d_v,
                     float *delta, uint32_t batch, uint32_t n_heads, uint32_t seq_len,
                     uint32_t d_head, float scale, uint32_t causal, void *stream) {
  DF_RANGE("df_attn_backward");
  int st = validate(batch, n_heads, seq_len, seq_len, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || seq_len == 0) return DF_OK;
  if (!q || !k || !v || !out || !d_out || !lse || !delta || !d_q || !d_k || !d_v) return finish(DF_ERR_INVALID_ARG);
  AttnParams p;
  p.q = q; p.k = k; p.v = v; p.o_in = out; p.d_out = d_out; p.lse_in = lse; p.delta = delta;
  p.d_q = d_q; p.d_k = d_k; p.d_v = d_v;
  p.B = batch; p.H = n_heads; p.Sq = seq_len; p.Sk = seq_len; p.D = d_head;
  p.scale = scale; p.causal = causal != 0; p.shift = 0;
  return finish(full_backward(p, static_cast<cudaStream_t>(stream)));
}

int df_attn_merge_partials(float *o_a, float *lse_a, const float *o_b, const float *lse_b,
                           uint32_t batch, uint32_t n_heads, uint32_t seq_len, uint32_t d_head,
                           void *stream) {
  int st = validate(batch, n_heads, seq_len, seq_len, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || seq_len == 0) return DF_OK;
  if (!o_a || !lse_a || !o_b || !lse_b) return finish(DF_ERR_INVALID_ARG);
  return finish(merge_partials(o_a, lse_a, o_b, lse_b, batch, n_heads, seq_len, d_head,
                               static_cast<cudaStream_t>(stream)));
}

int df_attn_accumulate(float *dst, const float *src, uint64_t n, void *stream) {
  if (n == 0) return DF_OK;
  if (!dst || !src) return finish(DF_ERR_INVALID_ARG);
  return finish(accumulate(dst, src, n, static_cast<cudaStream_t>(stream)));
}

// ---------------------------------------------------------------- projections around the attention op
namespace {
int linear_call(const float *x, const float *const *w, const float *const *bias, float *const *out, const float *residual,
                int n_mats, uint32_t rows, uint32_t in_features, uint32_t out_features, void *stream, float *gelu_out = nullptr) {
  if (rows == 0) return DF_OK;
  if (in_features == 0 || out_features == 0 || !x) return finish(DF_ERR_INVALID_ARG);
  for (int j = 0; j < n_mats; ++j)
    if (!w[j] || !out[j]) return finish(DF_ERR_INVALID_ARG);
  if ((uint64_t)rows * in_features >= (1ull << 40) || (uint64_t)rows * out_features >= (1ull << 40)) return finish(DF_ERR_INVALID_ARG);
  // tensor-core kernel only: there is no SIMT or CPU path behind these entry points
  if (!tensor_linear_supported(x, w, bias, out, residual, n_mats, rows, in_features, out_features)) return finish(DF_ERR_UNSUPPORTED);
  return finish(tensor_linear(x, w, bias, out, residual, gelu_out, n_mats, rows, in_features, out_features, static_cast<cudaStream_t>(stream)));
}
}  // namespace

int df_linear_qkv_forward(const float *x, const float *wq, const float *wk, const float *wv, const float *bq, const float *bk,
                          const float *bv, float *q, float *k, float *v, uint32_t rows, uint32_t in_features,
                          uint32_t out_features, void *stream) {
  DF_RANGE("df_linear_qkv_forward");
  const float *w[3] = {wq, wk, wv};
  const float *b[3] = {bq, bk, bv};
  float *o[3] = {q, k, v};
  const bool any_bias = bq || bk || bv;
  if (any_bias && !(bq && bk && bv)) return finish(DF_ERR_INVALID_ARG);
  return linear_call(x, w, any_bias ? b : nullptr, o, nullptr, 3, rows, in_features, out_features, stream);
}

int df_linear_forward(const float *x, const float *w, const float *bias, const float *residual, float *out, uint32_t rows,
                      uint32_t in_features, uint32_t out_features, void *stream) {
  DF_RANGE("df_linear_forward");
  const float *ws[1] = {w};
  const float *bs[1] = {bias};
  float *os[1] = {out};
  return linear_call(x, ws, bias ? bs : nullptr, os, residual, 1, rows, in_features, out_features, stream);
}

int df_linear_gelu_forward(const float *x, const float *w, const float *bias, float *pre_activation, float *out, uint32_t rows,
                           uint32_t in_features, uint32_t out_features, void *stream) {
  DF_RANGE("df_linear_gelu_forward");
  if (!out) return finish(DF_ERR_INVALID_ARG);
  const float *ws[1] = {w};
  const float *bs[1] = {bias};
  float *os[1] = {pre_activation ? pre_activation : out};  // no pre-activation wanted: the first output map is never stored through
  return linear_call(x, ws, bias ? bs : nullptr, os, nullptr, 1, rows, in_features, out_features, stream, out);
}

// ---------------------------------------------------------------- loss head
int df_chunked_logit_ce(float *logits, const uint32_t *targets, float *grad_logits, float *loss, uint32_t chunk_rows, uint32_t cols,
                        uint32_t total_rows, void *stream) {
  DF_RANGE("df_chunked_logit_ce");
  return finish(chunked_logit_ce(logits, targets, grad_logits, loss, chunk_rows, cols, total_rows, static_cast<cudaStream_t>(stream)));
}

void launch_fused_chunked_logit_ce(float *logits, const uint32_t *targets, float *grad_logits, float *loss, uint32_t chunk_rows,
                                   uint32_t cols, uint32_t total_rows) {
  if (!grad_logits) { finish(DF_ERR_INVALID_ARG); return; }
  df_chunked_logit_ce(logits, targets, grad_logits, loss, chunk_rows, cols, total_rows, nullptr);
}

void launch_chunked_ce_eval(float *logits, const uint32_t *targets, float *loss, uint32_t chunk_rows, uint32_t cols,
                            uint32_t total_rows) {
  df_chunked_logit_ce(logits, targets, nullptr, loss, chunk_rows, cols, total_rows, nullptr);
}

// ---------------------------------------------------------------- LayerNorm, GELU, AdamW of the training step
int df_layernorm_forward(const float *x, const float *gamma, const float *beta, float *out, float *means, float *rstds,
                         uint32_t rows, uint32_t cols, void *stream) {
  DF_RANGE("df_layernorm_forward");
  return finish(layernorm_forward(x, gamma, beta, out, means, rstds, rows, cols, static_cast<cudaStream_t>(stream)));
}
int df_layernorm_backward(const float *grad_out, const float *x, const float *gamma, const float *means, const float *rstds,
                          float *grad_x, float *grad_gamma, float *grad_beta, uint32_t rows, uint32_t cols, void *stream) {
  DF_RANGE("df_layernorm_backward");
  return finish(layernorm_backward(grad_out, x, gamma, means, rstds, grad_x, grad_gamma, grad_beta, rows, cols,
                                   static_cast<cudaStream_t>(stream)));
}
int df_gelu_forward(const float *x, float *out, uint64_t n, void *stream) {
  DF_RANGE("df_gelu_forward");
  return finish(gelu_forward(x, out, n, static_cast<cudaStream_t>(stream)));
}
int df_gelu_backward(const float *grad_out, const float *x, float *grad_x, uint64_t n, void *stream) {
  DF_RANGE("df_gelu_backward");
  return finish(gelu_backward(grad_out, x, grad_x, n, static_cast<cudaStream_t>(stream)));
}
int df_adamw_update(float *parameter, float *first_moment, float *second_moment, const float *gradient, uint64_t n, float lr,
                    float beta1, float beta2, float eps, float weight_decay, float bias_correction1, float bias_correction2,
                    void *stream) {
  DF_RANGE("df_adamw_update");
  return finish(adamw_update(parameter, first_moment, second_moment, gradient, n, lr, beta1, beta2, eps, weight_decay,
                             bias_correction1, bias_correction2, static_cast<cudaStream_t>(stream)));
}
uint64_t df_adamw_plan(df_adamw_tensor_t *tensors_host, uint32_t n_tensors) {
  return tensors_host ? adamw_plan(tensors_host, n_tensors) : 0;
}
int df_adamw_update_multi(const df_adamw_tensor_t *tensors_device, uint32_t n_tensors, uint64_t total_chunks, float lr, float beta1,
                          float beta2, float eps, float weight_decay, float bias_correction1, float bias_correction2,
                          void *stream) {
  DF_RANGE("df_adamw_update_multi");
  return finish(adamw_update_multi(tensors_device, n_tensors, total_chunks, lr, beta1, beta2, eps, weight_decay, bias_correction1,
                                   bias_correction2, static_cast<cudaStream_t>(stream)));
}
void launch_layernorm(const float *x, const float *gamma, const float *beta, float *out, float *means, float *rstds, uint32_t batch,
                      uint32_t features) {
  df_layernorm_forward(x, gamma, beta, out, means, rstds, batch, features, nullptr);
}
void launch_layernorm_backward(const float *grad_out, const float *x, const float *gamma, const float *means, const float *rstds,
                               float *grad_x, float *grad_gamma, float *grad_beta, uint32_t batch, uint32_t features) {
  df_layernorm_backward(grad_out, x, gamma, means, rstds, grad_x, grad_gamma, grad_beta, batch, features, nullptr);
}
void launch_gelu(const float *x, float *out, uint32_t n) { df_gelu_forward(x, out, n, nullptr); }
void launch_gelu_backward(const float *grad_out, const float *x, float *grad_x, uint32_t n) {
  df_gelu_backward(grad_out, x, grad_x, n, nullptr);
}
void launch_adamw_update(float *parameter, float *first_moment, float *second_moment, const float *gradient, uint32_t n, float lr,
                         float beta1, float beta2, float eps, float weight_decay, float bias_correction1,
                         float bias_correction2) {
  df_adamw_update(parameter, first_moment, second_moment, gradient, n, lr, beta1, beta2, eps, weight_decay, bias_correction1,
                  bias_correction2, nullptr);
}

// ---------------------------------------------------------------- one-time set-up and per-kernel timing
int df_attn_init(void) { return finish(tensor_backward_init()); }

int df_attn_backward_profile(const float *q, const float *k, const float *v, const float *out,
                             const float *d_out, const float *lse, float *d_q, float *d_k, float *d_v,
                             float *delta, uint32_t batch, uint32_t n_heads, uint32_t seq_len,
                             uint32_t d_head, float scale, uint32_t causal, void *stream, float *ms_dq,
                             float *ms_dkdv) {
  if (!ms_dq || !ms_dkdv) return finish(DF_ERR_INVALID_ARG);
  *ms_dq = *ms_dkdv = 0.0f;
  cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
  for (int i = 0; i < 3; ++i)
    if (check_cuda(cudaEventCreate(&ev[i])) != DF_OK) {
      for (int j = 0; j < i; ++j) cudaEventDestroy(ev[j]);
      return DF_ERR_CUDA;
    }
  tensor_backward_set_profile_events(ev);
  int st = df_attn_backward(q, k, v, out, d_out, lse, d_q, d_k, d_v, delta, batch, n_heads, seq_len, d_head, scale,
                            causal, stream);
  tensor_backward_set_profile_events(nullptr);
  if (st == DF_OK) st = check_cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (st == DF_OK && cudaEventQuery(ev[2]) == cudaSuccess) {  // the events were recorded: the tensor-core path ran
    if (cudaEventElapsedTime(ms_dq, ev[0], ev[1]) != cudaSuccess || cudaEventElapsedTime(ms_dkdv, ev[1], ev[2]) != cudaSuccess)
      *ms_dq = *ms_dkdv = 0.0f;
    *ms_dq /= (float)kProfileReps;
    *ms_dkdv /= (float)kProfileReps;
  }
  cudaGetLastError();  // an event that was never recorded reports an error above; it is not the caller's
  for (int i = 0; i < 3; ++i) cudaEventDestroy(ev[i]);
  return st;
}

// ---------------------------------------------------------------- backward without any scratch argument
// The delta row sums of this entry point live in a file-scope device array, so a caller that can
// neither allocate nor lend a buffer can still run the backward. In host code `g_static_delta`
// is only a handle for the runtime, not a device address: the address is looked up with
// cudaGetSymbolAddress once per device (with that device current) and that pointer is what the
// kernels receive.
namespace {
__device__ __align__(256) float g_static_delta[DF_STATIC_SCRATCH_MAX_ROWS];

float *static_delta_ptr() {
  constexpr int kMaxDev = 64;
  static float *cache[kMaxDev] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  float *ptr = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (!ptr) {
    void *addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_static_delta) != cudaSuccess || !addr) return nullptr;
    ptr = static_cast<float *>(addr);
    __atomic_store_n(&cache[dev], ptr, __ATOMIC_RELEASE);
  }
  return ptr;
}
}  // namespace

int df_attn_backward_static_scratch(const float *q, const float *k, const float *v, const float *out,
                                    const float *d_out, const float *lse, float *d_q, float *d_k,
                                    float *d_v, uint32_t batch, uint32_t n_heads, uint32_t seq_len,
                                    uint32_t d_head, float scale, uint32_t causal, void *stream) {
  DF_RANGE("df_attn_backward_static_scratch");
  int st = validate(batch, n_heads, seq_len, seq_len, d_head);
  if (st != DF_OK) return finish(st);
  if (batch == 0 || seq_len == 0) return DF_OK;
  if ((uint64_t)batch * n_heads * seq_len > (uint64_t)DF_STATIC_SCRATCH_MAX_ROWS)
    return finish(DF_ERR_STATIC_SCRATCH);  // refused before anything is launched
  if (!q || !k || !v || !out || !d_out || !lse || !d_q || !d_k || !d_v) return finish(DF_ERR_INVALID_ARG);
  float *delta = static_delta_ptr();  // first call on this device resolves the address
  if (!delta) return finish(DF_ERR_CUDA);
  // every row of delta that the backward kernels read is written first in the same call (by the
  // dQ kernel or the pre-pass), so stale contents from an earlier call are harmless and nothing
  // needs clearing
  AttnParams p;
  p.q = q; p.k = k; p.v = v; p.o_in = out; p.d_out = d_out; p.lse_in = lse; p.delta = delta;
  p.d_q = d_q; p.d_k = d_k; p.d_v = d_v;
  p.B = batch; p.H = n_heads; p.Sq = seq_len; p.Sk = seq_len; p.D = d_head;
  p.scale = scale; p.causal = causal != 0; p.shift = 0;
  return finish(full_backward(p, static_cast<cudaStream_t>(stream)));
}

// ---------------------------------------------------------------- scratch sizes (host only)
uint64_t df_attn_workspace_bytes(int kind, uint32_t batch, uint32_t n_heads, uint32_t seq_len, uint32_t d_head,
                                 uint32_t chunk_size) {
  const uint64_t B = batch, H = n_heads, S = seq_len, D = d_head;
  switch (kind) {
    case DF_WS_DELTA:          // `delta` of df_attn_backward / df_attn_delta: [B, H, S] floats
      return B * H * S * 4;
    case DF_WS_LSE:            // `lse` of df_attn_forward: [B, H, S] floats
      return B * H * S * 4;
    case DF_WS_LEGACY_BACKWARD:  // `probabilities` of launch_fused_mha_backward as the reference sizes it (lib.rs:2019-2027)
      return H * 2 * S * S * 4;
    case DF_WS_LEGACY_BACKWARD_MIN:  // what this library needs of it to stay on the tensor-core path: O, lse, delta
      return (S * H * D + 2 * H * S) * 4;
    case DF_WS_DECODE_PARTIALS: {  // partial_m + partial_l + partial_o of the split-K decode forms, in total
      if (chunk_size == 0) return 0;
      const uint64_t chunks = (S + chunk_size - 1) / chunk_size;
      return H * chunks * (2 + D) * 4;
    }
    default:
      return 0;
  }
}

// ---------------------------------------------------------------- schedule probe (host only)
long long df_attn_schedule_item(int round, int grid, int cta, long long n_items) {
  if (round < 0 || grid <= 0 || cta < 0 || cta >= grid || n_items < 0) return -1;
  return snake_item(round, grid, cta, n_items);
}

// ---------------------------------------------------------------- decode
int df_attn_decode(const float *q, const void *k, const void *v, const int32_t *block_table, float *out,
                   float *partial_m, float *partial_l, float *partial_o, uint32_t max_chunks,
                   uint32_t n_heads, uint32_t cur_seq_len, uint32_t d_head, float scale,
                   uint32_t page_size, uint32_t kv_bf16, void *stream) {
  DF_RANGE("df_attn_decode");
  if (d_head == 0 || d_head > 128 || n_heads == 0 || n_heads > 65535u) return finish(DF_ERR_INVALID_ARG);
  if (cur_seq_len == 0) return DF_OK;  // the reference kernels return without writing (attention_fused.cu:557)
  if (!q || !k || !v || !out) return finish(DF_ERR_INVALID_ARG);
  if (block_table && page_size == 0) return finish(DF_ERR_INVALID_ARG);
  if (!isfinite(scale)) return finish(DF_ERR_INVALID_ARG);
  return finish(decode_dispatch(q, k, v, block_table, out, partial_m, partial_l, partial_o, max_chunks, n_heads,
                                cur_seq_len, d_head, scale, page_size, kv_bf16 != 0, static_cast<cudaStream_t>(stream)));
}

void launch_fused_mha_decode_kv(const float *q, const float *k_cache, const float *v_cache, float *out,
                                uint32_t n_heads, uint32_t cur_seq_len, uint32_t d_head, float scale) {
  df_attn_decode(q, k_cache, v_cache, nullptr, out, nullptr, nullptr, nullptr, 0, n_heads, cur_seq_len, d_head, scale,
                 0, 0, nullptr);
}

void launch_fused_mha_decode_kv_splitk(const float *q, const float *k_cache, const float *v_cache,
                                       float *partial_m, float *partial_l, float *partial_o, float *out,
                                       uint32_t n_heads, uint32_t cur_seq_len, uint32_t d_head, float scale,
                                       uint32_t chunk_size) {
  const uint32_t chunks = chunk_size ? (cur_seq_len + chunk_size - 1) / chunk_size : 0;
  df_attn_decode(q, k_cache, v_cache, nullptr, out, partial_m, partial_l, partial_o, chunks, n_heads, cur_seq_len,
                 d_head, scale, 0, 0, nullptr);
}

void launch_paged_mha_decode_kv(const float *q, const float *k_pool, const float *v_pool,
                                const int32_t *block_table, float *out, uint32_t n_heads,
                                uint32_t cur_seq_len, uint32_t d_head, float scale, uint32_t page_size) {
  if (!block_table) { finish(DF_ERR_INVALID_ARG); return; }
  df_attn_decode(q, k_pool, v_pool, block_table, out, nullptr, nullptr, nullptr, 0, n_heads, cur_seq_len, d_head,
                 scale, page_size, 0, nullptr);
}

void launch_paged_mha_decode_kv_splitk(const float *q, const float *k_pool, const float *v_pool,
                                       const int32_t *block_table, float *partial_m, float *partial_l,
                                       float *partial_o, float *out, uint32_t n_heads, uint32_t cur_seq_len,
                                       uint32_t d_head, float scale, uint32_t page_size, uint32_t chunk_size) {
  if (!block_table) { finish(DF_ERR_INVALID_ARG); return; }
  const uint32_t chunks = chunk_size ? (cur_seq_len + chunk_size - 1) / chunk_size : 0;
  df_attn_decode(q, k_pool, v_pool, block_table, out, partial_m, partial_l, partial_o, chunks, n_heads, cur_seq_len,
                 d_head, scale, page_size, 0, nullptr);
}

void launch_paged_mha_decode_kv_bf16(const float *q, const void *k_pool, const void *v_pool,
                                     const int32_t *block_table, float *out, uint32_t n_heads,
                                     uint32_t cur_seq_len, uint32_t d_head, float scale, uint32_t page_size) {
  if (!block_table) { finish(DF_ERR_INVALID_ARG); return; }
  df_attn_decode(q, k_pool, v_pool, block_table, out, nullptr, nullptr, nullptr, 0, n_heads, cur_seq_len, d_head,
                 scale, page_size, 1, nullptr);
}

// ---------------------------------------------------------------- legacy symbols
void launch_fused_mha_forward(const float *q, const float *k, const float *v, float *out,
                              uint32_t n_heads, uint32_t seq_len, uint32_t d_head, float scale,
                              uint32_t causal) {
  df_attn_forward_block(q, k, v, out, nullptr, 1, n_heads, seq_len, seq_len, d_head, scale, causal,
                        0, nullptr);
}

void launch_fused_attention(const float *q, const float *k, const float *v, float *out,
                            uint32_t seq_len, uint32_t d_head, float scale, uint32_t causal) {
  df_attn_forward_block(q, k, v, out, nullptr, 1, 1, seq_len, seq_len, d_head, scale, causal, 0,
                        nullptr);
}

void launch_fused_mha_backward(const float *q, const float *k, const float *v, const float *d_out,
                               float *d_q, float *d_k, float *d_v, float *probabilities,
                               uint32_t n_heads, uint32_t seq_len, uint32_t d_head, float scale,
                               uint32_t causal) {
  finish(legacy_backward(q, k, v, d_out, d_q, d_k, d_v, probabilities,
                         2ull * n_heads * seq_len * seq_len, n_heads, seq_len, d_head, scale,
                         causal));
}

void launch_attention_backward(const float *q, const float *k, const float *v, const float *d_out,
                               float *d_q, float *d_k, float *d_v, float *probabilities,
                               uint32_t seq_len, uint32_t d_head, float scale, uint32_t causal) {
  finish(legacy_backward(q, k, v, d_out, d_q, d_k, d_v, probabilities,
                         (uint64_t)seq_len * seq_len, 1, seq_len, d_head, scale, causal));
}

int df_attn_selftest_wait_expiry(uint32_t budget_ms, void *stream) {
  if (budget_ms == 0 || budget_ms > 2000) return finish(DF_ERR_INVALID_ARG);
  unsigned int *status = device_status_ptr();
  if (!status) return finish(DF_ERR_CUDA);
  k_selftest_wait_expiry<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>((unsigned long long)budget_ms * 1000000ull, status);
  note_launch();
  return finish(check_cuda(cudaGetLastError()));
}

#ifdef DF_BOUNDS_CHECK
namespace df {
namespace {
// one thread asks the checker for element 5 of a 4-element tensor: the bit is set, element 0 is what it gets back
__device__ unsigned int g_bounds_selftest_seen;
__global__ void k_selftest_bounds(unsigned int *status) {
  g_bounds_selftest_seen = (unsigned int)DF_IDX(5, 4, status);
}
}  // namespace
}  // namespace df
#endif

int df_attn_selftest_bounds_check(void *stream) {
#ifdef DF_BOUNDS_CHECK
  unsigned int *status = df::device_status_ptr();
  if (!status) return df::finish(DF_ERR_CUDA);
  df::k_selftest_bounds<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(status);
  df::note_launch();
  return df::finish(df::check_cuda(cudaGetLastError()));
#else
  (void)stream;
  return DF_ERR_UNSUPPORTED;
#endif
}

int df_sync_status(void) {
  int st = check_cuda(cudaDeviceSynchronize());
  if (st == DF_OK) {
    unsigned int *w = device_status_ptr();
    unsigned int host = 0;
    if (w && cudaMemcpy(&host, w, sizeof(host), cudaMemcpyDeviceToHost) == cudaSuccess && host != 0) {
      cudaMemset(w, 0, sizeof(host));
      st = (host & DEV_STATUS_WAIT_EXPIRED) ? DF_ERR_DEVICE_TIMEOUT : DF_ERR_DEVICE_BOUNDS;
    }
  }
  return finish(st);
}

void darkforest_sync(void) {
  const int st = df_sync_status();
  if (st != DF_OK) fprintf(stderr, "darkforest_sync: %s\n", df_attn_status_string(st));
}

int df_attn_set_option(int which, int value) {
  if (which < 0 || which >= DF_OPT_COUNT) return -1;
  std::call_once(g_options_once, init_options);
  return g_options[which].exchange(value, std::memory_order_relaxed);
}

int df_attn_get_option(int which) { return (which < 0 || which >= DF_OPT_COUNT) ? -1 : option(which); }

int df_attn_set_variant(int variant) {
  const int prev = t_variant;
  if (variant >= DF_VARIANT_AUTO && variant <= DF_VARIANT_TENSOR) t_variant = variant;
  return prev;
}

int df_attn_forward_uses_tensor_cores(const void *q, const void *k, const void *v, const void *out,
                                      uint32_t n_heads, uint32_t seq_q, uint32_t seq_k,
                                      uint32_t d_head) {
  AttnParams p;
  p.q = static_cast<const float *>(q); p.k = static_cast<const float *>(k);
  p.v = static_cast<const float *>(v);
  p.out = const_cast<float *>(static_cast<const float *>(out));
  p.B = 1; p.H = n_heads; p.Sq = seq_q; p.Sk = seq_k; p.D = d_head;
  return (t_variant != DF_VARIANT_SIMT && tensor_forward_supported(p)) ? 1 : 0;
}

int df_attn_last_status(void) {
  const int s = t_status;
  t_status = DF_OK;
  return s;
}

const char *df_attn_status_string(int status) {
  switch (status) {
    case DF_OK: return "ok";
    case DF_ERR_INVALID_ARG: return "invalid argument";
    case DF_ERR_UNSUPPORTED: return "shape not supported by the selected variant";
    case DF_ERR_CUDA: return "CUDA call failed";
    case DF_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
    case DF_ERR_DEVICE_BOUNDS: return "a kernel of a DF_BOUNDS_CHECK build computed an index outside its tensor";
    case DF_ERR_WORKSPACE: return "caller scratch too small";
    case DF_ERR_STATIC_SCRATCH:
      return "batch*heads*seq_len exceeds DF_STATIC_SCRATCH_MAX_ROWS, the size of the built-in scratch array";
    case DF_ERR_RING_TIMEOUT: return "ring: a host-side wait on the communicator ran out and it was aborted";
    case DF_ERR_NCCL: return "ring: NCCL reported an error";
    default: return "unknown status";
  }
}

uint64_t df_attn_launch_count(int reset) {
  const uint64_t n = t_launches;
  if (reset) t_launches = 0;
  return n;
}

const char *df_attn_build_info(void) {
  return "darkforest_kernels for sm_100a (tcgen05/TMA attention + SIMT generic path), built " __DATE__;
}

}  // extern "C"
