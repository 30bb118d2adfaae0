// attention_context.hpp — C++ host layer over the attention library's C ABI.
//
// Mirrors the parts of darkforest-cuda's Rust wrapper layer that the attention path uses, with the
// same names, argument meaning and error behaviour, so that a caller of the reference finds what
// it expects:
//   DeviceTensor        darkforest-cuda/src/lib.rs:440-534  (zeros, as_ptr, as_mut_ptr, as_ptr_offset)
//   CudaEventTimer      lib.rs:157-224
//   cuda_sync           darkforest-cuda/src/kernels.rs:9-20  (returns a status instead of aborting)
//   get_memory_info     darkforest-cuda/src/memory.rs:40-53
//   AttentionContext    lib.rs:1949-2368: new / new_shared, forward_device_into, backward_device_into,
//                       forward_device, backward_device, host-slice forward / backward (single head)
// plus the calls the reference lacks: forward_lse_into / backward_from_lse_into (no S x S scratch).
// Errors are reported as df::Error exceptions carrying the reference's message texts.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/darkforest_kernels.h"

namespace df {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

inline void check_cuda(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw Error(std::string(what) + ": " + cudaGetErrorString(e));
}
inline void check_status(int st, const char *what) {
  if (st != DF_OK) throw Error(std::string(what) + ": " + df_attn_status_string(st));
}

// (free, total) bytes of the current device.
inline std::pair<size_t, size_t> get_memory_info() {
  size_t free_b = 0, total_b = 0;
  check_cuda(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo");
  return {free_b, total_b};
}

// Device synchronisation; throws instead of the reference's abort().
inline void cuda_sync() { check_status(df_sync_status(), "device synchronisation"); }

// Owning fp32 device tensor with a shape; every tensor is its own allocation, like the reference.
class DeviceTensor {
 public:
  DeviceTensor() = default;
  static DeviceTensor zeros(std::vector<size_t> shape) {
    DeviceTensor t;
    t.shape = std::move(shape);
    size_t n = 1;
    for (size_t d : t.shape) {
      if (d != 0 && n > SIZE_MAX / sizeof(float) / d) throw Error("tensor shape is too large");
      n *= d;
    }
    t.elems_ = n;
    if (n) {
      check_cuda(cudaMalloc(&t.ptr_, n * sizeof(float)), "cudaMalloc");
      check_cuda(cudaMemset(t.ptr_, 0, n * sizeof(float)), "cudaMemset");
    }
    return t;
  }
  static DeviceTensor from_host(const std::vector<float> &host, std::vector<size_t> shape) {
    DeviceTensor t = zeros(std::move(shape));
    if (host.size() != t.elems_) throw Error("host data does not match the tensor shape");
    if (t.elems_) check_cuda(cudaMemcpy(t.ptr_, host.data(), t.elems_ * sizeof(float), cudaMemcpyHostToDevice), "upload");
    return t;
  }
  DeviceTensor(DeviceTensor &&o) noexcept { *this = std::move(o); }
  DeviceTensor &operator=(DeviceTensor &&o) noexcept {
    if (this != &o) {
      release();
      shape = std::move(o.shape);
      ptr_ = o.ptr_;
      elems_ = o.elems_;
      o.ptr_ = nullptr;
      o.elems_ = 0;
    }
    return *this;
  }
  DeviceTensor(const DeviceTensor &) = delete;
  DeviceTensor &operator=(const DeviceTensor &) = delete;
  ~DeviceTensor() { release(); }

  const float *as_ptr() const { return ptr_; }
  float *as_mut_ptr() { return ptr_; }
  const float *as_ptr_offset(size_t elements) const { return ptr_ + elements; }
  size_t numel() const { return elems_; }
  std::vector<float> to_host() const {
    std::vector<float> h(elems_);
    if (elems_) check_cuda(cudaMemcpy(h.data(), ptr_, elems_ * sizeof(float), cudaMemcpyDeviceToHost), "download");
    return h;
  }
  std::vector<size_t> shape;

  // ---- the step's row-wise and elementwise methods of the reference's DeviceTensor, same names, argument order and
  // checks (darkforest-cuda/src/lib.rs:775-781 gelu_into, 894-910 gelu_backward_into, 1010-1040 layernorm_into,
  // 1074-1112 layernorm_backward_into, 1755-1787 adamw_update); they launch on the legacy stream like the reference.
  void zero_() {
    if (elems_) check_cuda(cudaMemsetAsync(ptr_, 0, elems_ * sizeof(float), nullptr), "cudaMemsetAsync");
  }
  void gelu_into(DeviceTensor &out) const {
    if (shape != out.shape) throw Error("DeviceTensor::gelu_into shape mismatch");
    check_status(df_gelu_forward(ptr_, out.ptr_, elems_, nullptr), "df_gelu_forward");
  }
  // self = the pre-activation input, like the reference: grad_x = grad_out * gelu'(self)
  void gelu_backward_into(const DeviceTensor &grad_out, DeviceTensor &grad_x) const {
    if (shape != grad_out.shape || shape != grad_x.shape) throw Error("gelu_backward_into shape mismatch");
    check_status(df_gelu_backward(grad_out.ptr_, ptr_, grad_x.ptr_, elems_, nullptr), "df_gelu_backward");
  }
  void layernorm_into(const DeviceTensor *gamma, const DeviceTensor *beta, DeviceTensor &out, DeviceTensor &means,
                      DeviceTensor &rstds) const {
    if (shape != out.shape) throw Error("layernorm_into output shape mismatch");
    if (shape.empty()) throw Error("layernorm empty shape");
    const size_t features = shape.back(), batch = features ? elems_ / features : 0;
    if (means.shape != std::vector<size_t>{batch} || rstds.shape != std::vector<size_t>{batch})
      throw Error("layernorm_into stats shape mismatch");
    if (batch > UINT32_MAX || features > UINT32_MAX) throw Error("layernorm_into: tensor too large");
    check_status(df_layernorm_forward(ptr_, gamma ? gamma->ptr_ : nullptr, beta ? beta->ptr_ : nullptr, out.ptr_, means.ptr_,
                                      rstds.ptr_, (uint32_t)batch, (uint32_t)features, nullptr),
                 "df_layernorm_forward");
  }
  // grad_gamma / grad_beta are zeroed first, as the reference does (the kernel adds to what they hold)
  static void layernorm_backward_into(const DeviceTensor &grad_out, const DeviceTensor &x, const DeviceTensor *gamma,
                                      const DeviceTensor &means, const DeviceTensor &rstds, DeviceTensor &grad_x,
                                      DeviceTensor *grad_gamma, DeviceTensor *grad_beta) {
    if (x.shape.empty()) throw Error("layernorm empty shape");
    const size_t features = x.shape.back(), batch = features ? x.elems_ / features : 0;
    if (grad_out.shape != x.shape || grad_x.shape != x.shape) throw Error("layernorm_backward_into shape mismatch");
    if (batch > UINT32_MAX || features > UINT32_MAX) throw Error("layernorm_backward_into: tensor too large");
    if (grad_gamma) grad_gamma->zero_();
    if (grad_beta) grad_beta->zero_();
    check_status(df_layernorm_backward(grad_out.ptr_, x.ptr_, gamma ? gamma->ptr_ : nullptr, means.ptr_, rstds.ptr_, grad_x.ptr_,
                                       grad_gamma ? grad_gamma->ptr_ : nullptr, grad_beta ? grad_beta->ptr_ : nullptr,
                                       (uint32_t)batch, (uint32_t)features, nullptr),
                 "df_layernorm_backward");
  }
  static void adamw_update(DeviceTensor &parameter, DeviceTensor &first_moment, DeviceTensor &second_moment,
                           const DeviceTensor &gradient, float lr, float beta1, float beta2, float eps, float weight_decay,
                           float bias_correction1, float bias_correction2) {
    if (parameter.shape != first_moment.shape || parameter.shape != second_moment.shape || parameter.shape != gradient.shape)
      throw Error("AdamW tensors must have matching shapes");
    check_status(df_adamw_update(parameter.ptr_, first_moment.ptr_, second_moment.ptr_, gradient.ptr_, parameter.elems_, lr, beta1,
                                 beta2, eps, weight_decay, bias_correction1, bias_correction2, nullptr),
                 "df_adamw_update");
  }

 private:
  void release() {
    if (ptr_) cudaFree(ptr_);
    ptr_ = nullptr;
  }
  float *ptr_ = nullptr;
  size_t elems_ = 0;
};

// Two events on the legacy stream, where the legacy launchers run.
class CudaEventTimer {
 public:
  CudaEventTimer() {
    check_cuda(cudaEventCreate(&start_), "cudaEventCreate");
    check_cuda(cudaEventCreate(&stop_), "cudaEventCreate");
  }
  ~CudaEventTimer() {
    cudaEventDestroy(start_);
    cudaEventDestroy(stop_);
  }
  CudaEventTimer(const CudaEventTimer &) = delete;
  CudaEventTimer &operator=(const CudaEventTimer &) = delete;
  void start() { check_cuda(cudaEventRecord(start_, 0), "cudaEventRecord"); }
  double stop_and_elapsed_ms() {
    check_cuda(cudaEventRecord(stop_, 0), "cudaEventRecord");
    check_cuda(cudaEventSynchronize(stop_), "cudaEventSynchronize");
    float ms = 0.f;
    check_cuda(cudaEventElapsedTime(&ms, start_, stop_), "cudaEventElapsedTime");
    return ms;
  }

 private:
  cudaEvent_t start_ = nullptr, stop_ = nullptr;
};

// Scratch shared between the layers of a model (the reference's Arc<Mutex<Option<CudaBuffer>>>,
// static_gpt2.rs:306, 401-406): allocated on the first backward, then reused.
struct SharedScratch {
  std::mutex mutex;
  float *ptr = nullptr;
  size_t floats = 0;
  ~SharedScratch() {
    if (ptr) cudaFree(ptr);
  }
};

class AttentionContext {
 public:
  const size_t n_heads, seq_len, d_head, d_model;

  AttentionContext(size_t heads, size_t seq, size_t dhead)
      : AttentionContext(heads, seq, dhead, std::make_shared<SharedScratch>()) {}
  // new_shared: several contexts (one per layer) share one scratch buffer.
  AttentionContext(size_t heads, size_t seq, size_t dhead, std::shared_ptr<SharedScratch> probabilities)
      : n_heads(heads), seq_len(seq), d_head(checked_d_head(dhead)), d_model(checked_mul(heads, dhead)),
        probabilities_(std::move(probabilities)) {
    checked_mul(seq, d_model);  // "attention shape is too large"
  }

  // ---- the reference's device-tensor API (legacy symbols, legacy stream, H*2*S*S scratch) ----
  void forward_device_into(const DeviceTensor &q, const DeviceTensor &k, const DeviceTensor &v, float scale, bool causal,
                           DeviceTensor &out) const {
    if (out.shape != std::vector<size_t>{seq_len, d_model}) throw Error("attention output shape mismatch");
    if (n_heads == 1)
      launch_fused_attention(q.as_ptr(), k.as_ptr(), v.as_ptr(), out.as_mut_ptr(), (uint32_t)seq_len, (uint32_t)d_head, scale,
                             causal);
    else
      launch_fused_mha_forward(q.as_ptr(), k.as_ptr(), v.as_ptr(), out.as_mut_ptr(), (uint32_t)n_heads, (uint32_t)seq_len,
                               (uint32_t)d_head, scale, causal);
    check_status(df_attn_last_status(), "attention forward");
  }
  DeviceTensor forward_device(const DeviceTensor &q, const DeviceTensor &k, const DeviceTensor &v, float scale,
                              bool causal) const {
    DeviceTensor out = DeviceTensor::zeros({seq_len, d_model});
    forward_device_into(q, k, v, scale, causal, out);
    return out;
  }
  void backward_device_into(const DeviceTensor &q, const DeviceTensor &k, const DeviceTensor &v, const DeviceTensor &d_out,
                            float scale, bool causal, DeviceTensor &d_q, DeviceTensor &d_k, DeviceTensor &d_v) const {
    const std::vector<size_t> want{seq_len, d_model};
    if (d_q.shape != want || d_k.shape != want || d_v.shape != want) throw Error("attention gradient shape mismatch");
    float *scratch = ensure_probabilities();
    if (n_heads == 1)
      launch_attention_backward(q.as_ptr(), k.as_ptr(), v.as_ptr(), d_out.as_ptr(), d_q.as_mut_ptr(), d_k.as_mut_ptr(),
                                d_v.as_mut_ptr(), scratch, (uint32_t)seq_len, (uint32_t)d_head, scale, causal);
    else
      launch_fused_mha_backward(q.as_ptr(), k.as_ptr(), v.as_ptr(), d_out.as_ptr(), d_q.as_mut_ptr(), d_k.as_mut_ptr(),
                                d_v.as_mut_ptr(), scratch, (uint32_t)n_heads, (uint32_t)seq_len, (uint32_t)d_head, scale,
                                causal);
    check_status(df_attn_last_status(), "attention backward");
  }

  // ---- what the reference lacks: logsumexp-saving forward, backward without the S x S scratch ----
  // lse and delta are caller-owned [n_heads, seq_len] tensors.
  void forward_lse_into(const DeviceTensor &q, const DeviceTensor &k, const DeviceTensor &v, float scale, bool causal,
                        DeviceTensor &out, DeviceTensor &lse, cudaStream_t stream = nullptr) const {
    check_status(df_attn_forward(q.as_ptr(), k.as_ptr(), v.as_ptr(), out.as_mut_ptr(), lse.as_mut_ptr(), 1, (uint32_t)n_heads,
                                 (uint32_t)seq_len, (uint32_t)d_head, scale, causal, stream),
                 "attention forward");
  }
  void backward_from_lse_into(const DeviceTensor &q, const DeviceTensor &k, const DeviceTensor &v, const DeviceTensor &out,
                              const DeviceTensor &d_out, const DeviceTensor &lse, float scale, bool causal, DeviceTensor &d_q,
                              DeviceTensor &d_k, DeviceTensor &d_v, DeviceTensor &delta, cudaStream_t stream = nullptr) const {
    check_status(df_attn_backward(q.as_ptr(), k.as_ptr(), v.as_ptr(), out.as_ptr(), d_out.as_ptr(), lse.as_ptr(),
                                  d_q.as_mut_ptr(), d_k.as_mut_ptr(), d_v.as_mut_ptr(), delta.as_mut_ptr(), 1,
                                  (uint32_t)n_heads, (uint32_t)seq_len, (uint32_t)d_head, scale, causal, stream),
                 "attention backward");
  }

  // ---- decode: one query token over a KV cache (lib.rs:2089-2222), legacy symbols, legacy stream ----
  // q, out: [d_model]; k_cache, v_cache: [max_seq_len, d_model]; the first cur_seq_len rows are attended.
  void decode_kv_into(const DeviceTensor &q, const DeviceTensor &k_cache, const DeviceTensor &v_cache, size_t cur_seq_len,
                      float scale, DeviceTensor &out) const {
    if (q.numel() != d_model || out.numel() != d_model) throw Error("decode_kv_into Q or Out dimension mismatch");
    if (cur_seq_len == 0 || k_cache.shape.empty() || cur_seq_len > k_cache.shape[0])
      throw Error("decode_kv_into cur_seq_len out of bounds");
    launch_fused_mha_decode_kv(q.as_ptr(), k_cache.as_ptr(), v_cache.as_ptr(), out.as_mut_ptr(), (uint32_t)n_heads,
                               (uint32_t)cur_seq_len, (uint32_t)d_head, scale);
    check_status(df_attn_last_status(), "attention decode");
  }
  // k_pool, v_pool: pages of page_size rows of d_model floats; block_table: device int32, one entry per logical page.
  void decode_paged_kv_into(const DeviceTensor &q, const DeviceTensor &k_pool, const DeviceTensor &v_pool,
                            const int32_t *block_table, size_t cur_seq_len, float scale, size_t page_size,
                            DeviceTensor &out) const {
    if (q.numel() != d_model || out.numel() != d_model) throw Error("decode_paged_kv_into Q or Out dimension mismatch");
    if (cur_seq_len == 0) return;
    launch_paged_mha_decode_kv(q.as_ptr(), k_pool.as_ptr(), v_pool.as_ptr(), block_table, out.as_mut_ptr(), (uint32_t)n_heads,
                               (uint32_t)cur_seq_len, (uint32_t)d_head, scale, (uint32_t)page_size);
    check_status(df_attn_last_status(), "paged attention decode");
  }
  // partial_m, partial_l: [n_heads * chunks], partial_o: [n_heads * chunks * d_head], chunks = ceil(cur_seq_len / chunk_size)
  void decode_paged_kv_splitk_into(const DeviceTensor &q, const DeviceTensor &k_pool, const DeviceTensor &v_pool,
                                   const int32_t *block_table, DeviceTensor &partial_m, DeviceTensor &partial_l,
                                   DeviceTensor &partial_o, size_t cur_seq_len, float scale, size_t page_size,
                                   size_t chunk_size, DeviceTensor &out) const {
    if (q.numel() != d_model || out.numel() != d_model)
      throw Error("decode_paged_kv_splitk_into Q or Out dimension mismatch");
    if (cur_seq_len == 0) return;
    launch_paged_mha_decode_kv_splitk(q.as_ptr(), k_pool.as_ptr(), v_pool.as_ptr(), block_table, partial_m.as_mut_ptr(),
                                      partial_l.as_mut_ptr(), partial_o.as_mut_ptr(), out.as_mut_ptr(), (uint32_t)n_heads,
                                      (uint32_t)cur_seq_len, (uint32_t)d_head, scale, (uint32_t)page_size,
                                      (uint32_t)chunk_size);
    check_status(df_attn_last_status(), "paged split-K attention decode");
  }

  // ---- host-slice variants (single head only, lib.rs:2295-2367): upload, run, download ----
  std::vector<float> forward(const std::vector<float> &q, const std::vector<float> &k, const std::vector<float> &v,
                             float scale, bool causal) const {
    if (n_heads != 1) throw Error("host-slice attention is single-head only");
    const std::vector<size_t> shape{seq_len, d_model};
    DeviceTensor dq = DeviceTensor::from_host(q, shape), dk = DeviceTensor::from_host(k, shape),
                 dv = DeviceTensor::from_host(v, shape);
    DeviceTensor out = forward_device(dq, dk, dv, scale, causal);
    cuda_sync();
    return out.to_host();
  }
  struct Gradients {
    std::vector<float> d_q, d_k, d_v;
  };
  Gradients backward(const std::vector<float> &q, const std::vector<float> &k, const std::vector<float> &v,
                     const std::vector<float> &d_out, float scale, bool causal) const {
    if (n_heads != 1) throw Error("host-slice attention is single-head only");
    const std::vector<size_t> shape{seq_len, d_model};
    DeviceTensor dq = DeviceTensor::from_host(q, shape), dk = DeviceTensor::from_host(k, shape),
                 dv = DeviceTensor::from_host(v, shape), dg = DeviceTensor::from_host(d_out, shape);
    DeviceTensor gq = DeviceTensor::zeros(shape), gk = DeviceTensor::zeros(shape), gv = DeviceTensor::zeros(shape);
    backward_device_into(dq, dk, dv, dg, scale, causal, gq, gk, gv);
    cuda_sync();
    return {gq.to_host(), gk.to_host(), gv.to_host()};
  }

 private:
  static size_t checked_d_head(size_t d) {
    if (d == 0 || d > 128) throw Error("d_head must be in the range 1..=128");  // lib.rs:1981
    return d;
  }
  static size_t checked_mul(size_t a, size_t b) {
    if (a != 0 && b > SIZE_MAX / a) throw Error("attention shape is too large");
    return a * b;
  }
  // First backward allocates n_heads*2*S*S floats like the reference (lib.rs:2019-2027).
  float *ensure_probabilities() const {
    std::lock_guard<std::mutex> guard(probabilities_->mutex);
    const size_t want = checked_mul(checked_mul(n_heads * 2, seq_len), seq_len);
    if (!probabilities_->ptr || probabilities_->floats < want) {
      if (probabilities_->ptr) cudaFree(probabilities_->ptr);
      probabilities_->ptr = nullptr;
      check_cuda(cudaMalloc(&probabilities_->ptr, (want ? want : 1) * sizeof(float)), "cudaMalloc(probabilities)");
      probabilities_->floats = want;
    }
    return probabilities_->ptr;
  }
  std::shared_ptr<SharedScratch> probabilities_;
};

// Free functions of the reference (lib.rs:2371-2479).
inline std::vector<float> fused_attention_forward(const std::vector<float> &q, const std::vector<float> &k,
                                                  const std::vector<float> &v, size_t seq_len, size_t d_head, float scale,
                                                  bool causal) {
  return AttentionContext(1, seq_len, d_head).forward(q, k, v, scale, causal);
}
inline AttentionContext::Gradients attention_backward(const std::vector<float> &q, const std::vector<float> &k,
                                                      const std::vector<float> &v, const std::vector<float> &d_out,
                                                      size_t seq_len, size_t d_head, float scale, bool causal) {
  return AttentionContext(1, seq_len, d_head).backward(q, k, v, d_out, scale, causal);
}

}  // namespace df
