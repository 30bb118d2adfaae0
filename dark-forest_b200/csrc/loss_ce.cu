// loss_ce.cu — the loss head's fused softmax + cross-entropy over one chunk of logits, for B200 (sm_100a).
//
// Drop-in for two symbols of darkforest-cuda/kernels/softmax.cu, which the reference's static step calls once per
// 512-row chunk of the vocabulary logits (darkforest-core/src/engine/static_gpt2.rs:1386-1418 through
// darkforest-cuda/src/lib.rs:1897-1945 and src/kernels.rs:531-600):
//   launch_fused_chunked_logit_ce  (softmax.cu:325-410)  logits -> probabilities in place, grad_logits =
//                                  (p - onehot(target)) / total_rows, loss += sum_rows -log(max(p_target, 1e-12)) / total_rows
//   launch_chunked_ce_eval         (softmax.cu:415-480)  loss += sum_rows (log(sum) - (z_target - max)) / total_rows
// Same arithmetic (max-subtracted softmax in fp32 with __expf / __logf); what differs is the traffic. The
// reference walks each row of [chunk_rows, vocab] three times through global memory (max; exp + write; normalise +
// two writes: 3 reads, 3 writes of the 200 KB row). Here a CTA keeps the whole row in shared memory (a 50257-entry
// row is 201 KB of the 227 KB an SM offers), so the training form reads the logits once and writes probabilities
// and gradients once each (1 read + 2 writes, the algorithmic minimum), and the eval form reads once with an online
// (max, sum) pair and writes nothing. The kernels are HBM-bound; grids are persistent (one CTA per SM, rows dealt
// round robin). Rows of an odd-length vocabulary are not 16-byte aligned: every row is processed as a scalar head up
// to the next 16-byte boundary, a float4 body and a scalar tail. Rows too long for shared memory take a two-pass
// form from global memory (online max/sum, then the write pass).
#include <float.h>
#include <math.h>

#include <mutex>

#include "df_common.cuh"

namespace df {
namespace {

constexpr int kCeThreads = 1024;
constexpr uint32_t kMaxSmemCols = 56 * 1024;  // 224 KB of floats: 57344 entries

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Block-wide reductions over kCeThreads threads; `red` holds 32 floats. Every thread gets the result.
__device__ __forceinline__ float block_max(float v, float *red) {
  v = warp_max(v);
  __syncthreads();  // the previous use of `red` is over
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[threadIdx.x & 31];  // kCeThreads / 32 = 32 warps: every slot is written
  return warp_max(r);
}
__device__ __forceinline__ float block_sum(float v, float *red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[threadIdx.x & 31];
  return warp_sum(r);
}

// [0, head) scalar, [head, head + 4 * n4) as float4, rest scalar: `head` elements bring the row to a 16-byte boundary
__device__ __forceinline__ void split_row(const float *row, uint32_t cols, uint32_t *head, uint32_t *n4) {
  const uint32_t mis = (uint32_t)((reinterpret_cast<uintptr_t>(row) >> 2) & 3u);
  uint32_t h = (4u - mis) & 3u;
  if (h > cols) h = cols;
  *head = h;
  *n4 = (cols - h) >> 2;
}

// Training form, row resident in shared memory.
__global__ void __launch_bounds__(kCeThreads, 1)
k_chunked_logit_ce_smem(float *__restrict__ logits, const uint32_t *__restrict__ targets, float *__restrict__ grad_logits,
                        float *__restrict__ loss, uint32_t chunk_rows, uint32_t cols, float inv_total_rows) {
  extern __shared__ __align__(16) float srow[];  // cols floats (+ up to 3 of padding in front), then 32 reduction slots
  float *red = srow + ((cols + 3u + 3u) & ~3u);
  float cta_loss = 0.0f;
  for (uint32_t row = blockIdx.x; row < chunk_rows; row += gridDim.x) {
    float *grow = logits + (size_t)row * cols;
    float *ggrad = grad_logits + (size_t)row * cols;
    const uint32_t target = __ldg(targets + row);
    uint32_t head, n4;
    split_row(grow, cols, &head, &n4);
    // the shared copy is shifted so that the float4 body is 16-byte aligned on both sides
    float *s = srow + ((4u - head) & 3u);
    const uint32_t body_end = head + 4u * n4;
    // ---- pass 1: global -> shared, running maximum
    float tmax = -FLT_MAX;
    if (threadIdx.x < head) {
      const float x = grow[threadIdx.x];
      s[threadIdx.x] = x;
      tmax = x;
    }
    {
      const float4 *g4 = reinterpret_cast<const float4 *>(grow + head);
      float4 *s4 = reinterpret_cast<float4 *>(s + head);
#pragma unroll 4
      for (uint32_t i = threadIdx.x; i < n4; i += kCeThreads) {
        const float4 x = __ldcs(g4 + i);  // read once: do not keep it in L2
        s4[i] = x;
        tmax = fmaxf(tmax, fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w)));
      }
    }
    if (body_end + threadIdx.x < cols) {
      const float x = grow[body_end + threadIdx.x];
      s[body_end + threadIdx.x] = x;
      tmax = fmaxf(tmax, x);
    }
    const float row_max = block_max(tmax, red);
    // ---- pass 2 (shared memory only): e = exp(x - max), sum
    float tsum = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += kCeThreads) {
      const float e = __expf(s[i] - row_max);
      s[i] = e;
      tsum += e;
    }
    const float inv_sum = 1.0f / block_sum(tsum, red);
    // ---- pass 3: probabilities and gradients out (streaming stores)
    const float g_scale = inv_total_rows;
    auto emit = [&](uint32_t i) {
      const float p = s[i] * inv_sum;
      grow[i] = p;
      ggrad[i] = (p - (i == target ? 1.0f : 0.0f)) * g_scale;
    };
    if (threadIdx.x < head) emit(threadIdx.x);
    {
      float4 *g4 = reinterpret_cast<float4 *>(grow + head);
      float4 *d4 = reinterpret_cast<float4 *>(ggrad + head);  // same 16-byte phase as the logits row (the launcher checks)
      const float4 *s4 = reinterpret_cast<const float4 *>(s + head);
#pragma unroll 4
      for (uint32_t i = threadIdx.x; i < n4; i += kCeThreads) {
        float4 p = s4[i];
        p.x *= inv_sum; p.y *= inv_sum; p.z *= inv_sum; p.w *= inv_sum;
        __stcs(g4 + i, p);
        // the target column (if it lies in this group of four) takes the scalar formula, (p - 1) * scale
        const uint32_t k = target - (head + 4u * i);  // unsigned: 4 or more when the target is elsewhere
        const float4 g = make_float4((p.x - (k == 0u ? 1.0f : 0.0f)) * g_scale, (p.y - (k == 1u ? 1.0f : 0.0f)) * g_scale,
                                     (p.z - (k == 2u ? 1.0f : 0.0f)) * g_scale, (p.w - (k == 3u ? 1.0f : 0.0f)) * g_scale);
        __stcs(d4 + i, g);
      }
    }
    if (body_end + threadIdx.x < cols) emit(body_end + threadIdx.x);
    if (threadIdx.x == 0 && target < cols) cta_loss += -__logf(fmaxf(s[target] * inv_sum, 1e-12f)) * inv_total_rows;
    __syncthreads();  // the row buffer is reused by the next row
  }
  if (threadIdx.x == 0 && cta_loss != 0.0f) atomicAdd(loss, cta_loss);
}

// Training form for rows that do not fit shared memory: online (max, sum) pass, then the write pass.
__global__ void __launch_bounds__(kCeThreads, 1)
k_chunked_logit_ce_global(float *__restrict__ logits, const uint32_t *__restrict__ targets, float *__restrict__ grad_logits,
                          float *__restrict__ loss, uint32_t chunk_rows, uint32_t cols, float inv_total_rows) {
  __shared__ float red[32];
  float cta_loss = 0.0f;
  for (uint32_t row = blockIdx.x; row < chunk_rows; row += gridDim.x) {
    float *grow = logits + (size_t)row * cols;
    float *ggrad = grad_logits + (size_t)row * cols;
    const uint32_t target = __ldg(targets + row);
    float tmax = -FLT_MAX;
    for (uint32_t i = threadIdx.x; i < cols; i += kCeThreads) tmax = fmaxf(tmax, grow[i]);
    const float row_max = block_max(tmax, red);
    float tsum = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += kCeThreads) tsum += __expf(grow[i] - row_max);
    const float inv_sum = 1.0f / block_sum(tsum, red);
    for (uint32_t i = threadIdx.x; i < cols; i += kCeThreads) {
      const float p = __expf(grow[i] - row_max) * inv_sum;
      grow[i] = p;
      ggrad[i] = (p - (i == target ? 1.0f : 0.0f)) * inv_total_rows;
      if (i == target) cta_loss += -__logf(fmaxf(p, 1e-12f)) * inv_total_rows;
    }
  }
  cta_loss = block_sum(cta_loss, red);
  if (threadIdx.x == 0 && cta_loss != 0.0f) atomicAdd(loss, cta_loss);
}

// Training form without a resident row: one CTA per row, several CTAs per SM. Pass 1 reads the row from DRAM with an
// online (max, sum) per thread; pass 2 reads it again - out of L2, where a 200 KB row of a 100 MB chunk still sits a few
// microseconds later - and writes probabilities and gradients with streaming stores. DRAM traffic is the same 1 read
// + 2 writes as the resident-row kernel; what it buys is overlap: with three CTAs per SM, one row's loads run under
// another row's stores, where a CTA that owns the whole SM alternates between them. Measured on B200 (512 x 50257):
// 0.075-0.077 ms against 0.078 ms for the resident-row kernel - both sit at 4.0-4.1 TB/s of algorithmic traffic, which
// looks like what HBM gives a one-read-two-writes stream - so the resident-row kernel (one loss atomic per CTA) stays
// the default and this one is selectable (DF_OPT_CE_VARIANT = 2).
constexpr int kCeL2Threads = 512;
__global__ void __launch_bounds__(kCeL2Threads, 3)
k_chunked_logit_ce_l2(float *__restrict__ logits, const uint32_t *__restrict__ targets, float *__restrict__ grad_logits,
                      float *__restrict__ loss, uint32_t chunk_rows, uint32_t cols, float inv_total_rows) {
  __shared__ float red[32];
  const uint32_t row = blockIdx.x;
  if (row >= chunk_rows) return;
  float *grow = logits + (size_t)row * cols;
  float *ggrad = grad_logits + (size_t)row * cols;
  const uint32_t target = __ldg(targets + row);
  uint32_t head, n4;
  split_row(grow, cols, &head, &n4);
  const uint32_t body_end = head + 4u * n4;
  const int n_warps = kCeL2Threads / 32;
  auto reduce = [&](float v, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = (int)(threadIdx.x & 31) < n_warps ? red[threadIdx.x & 31] : (is_max ? -FLT_MAX : 0.0f);
    return is_max ? warp_max(r) : warp_sum(r);
  };
  // ---- pass 1: online (max, sum)
  float m = -FLT_MAX, sm = 0.0f;
  auto push = [&](float x) {
    if (x > m) {
      sm = sm * __expf(m - x) + 1.0f;
      m = x;
    } else {
      sm += __expf(x - m);
    }
  };
  if (threadIdx.x < head) push(grow[threadIdx.x]);
  {
    const float4 *g4 = reinterpret_cast<const float4 *>(grow + head);
#pragma unroll 4
    for (uint32_t i = threadIdx.x; i < n4; i += kCeL2Threads) {
      const float4 x = g4[i];  // default caching: the row is wanted again in pass 2
      const float gm = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
      if (gm > m) {
        sm *= __expf(m - gm);
        m = gm;
      }
      sm += __expf(x.x - m) + __expf(x.y - m) + __expf(x.z - m) + __expf(x.w - m);
    }
  }
  if (body_end + threadIdx.x < cols) push(grow[body_end + threadIdx.x]);
  const float row_max = reduce(m, true);
  const float inv_sum = 1.0f / reduce(sm * __expf(m - row_max), false);
  // ---- pass 2: probabilities and gradients
  const float g_scale = inv_total_rows;
  auto emit = [&](uint32_t i) {
    const float p = __expf(grow[i] - row_max) * inv_sum;
    grow[i] = p;
    ggrad[i] = (p - (i == target ? 1.0f : 0.0f)) * g_scale;
    if (i == target) atomicAdd(loss, -__logf(fmaxf(p, 1e-12f)) * inv_total_rows);
  };
  if (threadIdx.x < head) emit(threadIdx.x);
  {
    float4 *g4 = reinterpret_cast<float4 *>(grow + head);
    float4 *d4 = reinterpret_cast<float4 *>(ggrad + head);
#pragma unroll 4
    for (uint32_t i = threadIdx.x; i < n4; i += kCeL2Threads) {
      const float4 x = g4[i];
      float4 p;
      p.x = __expf(x.x - row_max) * inv_sum; p.y = __expf(x.y - row_max) * inv_sum;
      p.z = __expf(x.z - row_max) * inv_sum; p.w = __expf(x.w - row_max) * inv_sum;
      __stcs(g4 + i, p);
      const uint32_t k = target - (head + 4u * i);
      const float4 g = make_float4((p.x - (k == 0u ? 1.0f : 0.0f)) * g_scale, (p.y - (k == 1u ? 1.0f : 0.0f)) * g_scale,
                                   (p.z - (k == 2u ? 1.0f : 0.0f)) * g_scale, (p.w - (k == 3u ? 1.0f : 0.0f)) * g_scale);
      __stcs(d4 + i, g);
      if (k < 4u) {
        const float pt = k == 0u ? p.x : (k == 1u ? p.y : (k == 2u ? p.z : p.w));
        atomicAdd(loss, -__logf(fmaxf(pt, 1e-12f)) * inv_total_rows);
      }
    }
  }
  if (body_end + threadIdx.x < cols) emit(body_end + threadIdx.x);
}

// Eval form: one read of the row, online (max, sum) per thread, nothing written but the loss. One row per CTA, four
// CTAs per SM.
__global__ void __launch_bounds__(kCeL2Threads, 4)
k_chunked_ce_eval(const float *__restrict__ logits, const uint32_t *__restrict__ targets, float *__restrict__ loss,
                  uint32_t chunk_rows, uint32_t cols, float inv_total_rows) {
  __shared__ float red[32];
  const uint32_t row = blockIdx.x;
  if (row >= chunk_rows) return;
  const float *grow = logits + (size_t)row * cols;
  const uint32_t target = __ldg(targets + row);
  uint32_t head, n4;
  split_row(grow, cols, &head, &n4);
  const uint32_t body_end = head + 4u * n4;
  const int n_warps = kCeL2Threads / 32;
  auto reduce = [&](float v, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = (int)(threadIdx.x & 31) < n_warps ? red[threadIdx.x & 31] : (is_max ? -FLT_MAX : 0.0f);
    return is_max ? warp_max(r) : warp_sum(r);
  };
  float m = -FLT_MAX, s = 0.0f;
  auto push = [&](float x) {
    if (x > m) {
      s = s * __expf(m - x) + 1.0f;
      m = x;
    } else {
      s += __expf(x - m);
    }
  };
  if (threadIdx.x < head) push(grow[threadIdx.x]);
  const float4 *g4 = reinterpret_cast<const float4 *>(grow + head);
#pragma unroll 4
  for (uint32_t i = threadIdx.x; i < n4; i += kCeL2Threads) {
    const float4 x = __ldcs(g4 + i);
    const float gm = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
    if (gm > m) {
      s *= __expf(m - gm);
      m = gm;
    }
    s += __expf(x.x - m) + __expf(x.y - m) + __expf(x.z - m) + __expf(x.w - m);
  }
  if (body_end + threadIdx.x < cols) push(grow[body_end + threadIdx.x]);
  const float row_max = reduce(m, true);
  const float sum = reduce(s * __expf(m - row_max), false);  // a thread that saw nothing has s = 0
  if (threadIdx.x == 0 && target < cols)
    atomicAdd(loss, (-(grow[target] - row_max) + __logf(fmaxf(sum, 1e-12f))) * inv_total_rows);
}

struct DeviceInfo {
  std::once_flag once;
  int n_sm = 0;
  bool ok = false;
};
DeviceInfo g_dev[64];

int device_info(int *n_sm) {
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev)) != DF_OK || dev < 0 || dev >= 64) return DF_ERR_CUDA;
  DeviceInfo &d = g_dev[dev];
  std::call_once(d.once, [&]() {
    d.ok = cudaFuncSetAttribute(k_chunked_logit_ce_smem, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess &&
           cudaDeviceGetAttribute(&d.n_sm, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && d.n_sm > 0;
  });
  if (!d.ok) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  *n_sm = d.n_sm;
  return DF_OK;
}

}  // namespace

int chunked_logit_ce(float *logits, const uint32_t *targets, float *grad_logits, float *loss, uint32_t chunk_rows, uint32_t cols,
                     uint32_t total_rows, cudaStream_t s) {
  if (chunk_rows == 0 || cols == 0) return DF_OK;
  if (!logits || !targets || !loss || total_rows == 0) return DF_ERR_INVALID_ARG;
  int n_sm = 0;
  if (device_info(&n_sm) != DF_OK) return DF_ERR_CUDA;
  const unsigned grid = chunk_rows < (uint32_t)n_sm ? chunk_rows : (unsigned)n_sm;
  const float inv = 1.0f / (float)total_rows;
  if (!grad_logits) {
    k_chunked_ce_eval<<<chunk_rows, kCeL2Threads, 0, s>>>(logits, targets, loss, chunk_rows, cols, inv);
    note_launch();
    return check_cuda(cudaGetLastError());
  }
  // the vector path of the resident-row kernel needs logits and grad_logits rows to be misaligned alike
  const bool same_phase = ((reinterpret_cast<uintptr_t>(logits) ^ reinterpret_cast<uintptr_t>(grad_logits)) & 15u) == 0 &&
                          (reinterpret_cast<uintptr_t>(logits) & 3u) == 0;
  // DF_OPT_CE_VARIANT: 0 / 1 = resident row (default), 2 = two passes with the second out of L2
  const int variant = option(DF_OPT_CE_VARIANT);
  if (same_phase && variant == 2) {
    k_chunked_logit_ce_l2<<<chunk_rows, kCeL2Threads, 0, s>>>(logits, targets, grad_logits, loss, chunk_rows, cols, inv);
    note_launch();
    return check_cuda(cudaGetLastError());
  }
  if (cols <= kMaxSmemCols && same_phase) {
    const size_t smem = ((size_t)((cols + 6u) & ~3u) + 32) * sizeof(float);
    k_chunked_logit_ce_smem<<<grid, kCeThreads, smem, s>>>(logits, targets, grad_logits, loss, chunk_rows, cols, inv);
    note_launch();
    return check_cuda(cudaGetLastError());
  }
  k_chunked_logit_ce_global<<<grid, kCeThreads, 0, s>>>(logits, targets, grad_logits, loss, chunk_rows, cols, inv);
  note_launch();
  return check_cuda(cudaGetLastError());
}

}  // namespace df
