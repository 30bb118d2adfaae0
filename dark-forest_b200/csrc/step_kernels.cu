// step_kernels.cu — the elementwise and row-wise kernels of the training step around attention, for B200 (sm_100a):
// LayerNorm forward / backward, GELU forward / backward and the AdamW update.
//
// Drop-in for five symbols the reference's static step calls on every layer and every parameter tensor
// (darkforest-core/src/engine/static_gpt2.rs:1314-1364 forward, :1426-1500 backward, :1651-1700 optimiser, through
// darkforest-cuda/src/lib.rs:769-790, 885-910, 993-1100, 1755-1800):
//   launch_layernorm           (kernels/layernorm.cu:97-108)     out = (x - mean) * rstd * gamma + beta, mean and rstd kept
//   launch_layernorm_backward  (kernels/layernorm.cu:187-200)    grad_x; grad_gamma and grad_beta ACCUMULATED into the caller's buffers
//   launch_gelu                (kernels/elementwise.cu:195-199)  tanh form
//   launch_gelu_backward       (kernels/elementwise.cu:217-224)
//   launch_adamw_update        (kernels/matmul.cu:341-363)       decoupled weight decay, bias corrections passed in
// Same arithmetic; what differs is the traffic and the number of launches. All five are HBM-bound.
//  * LayerNorm: the reference runs one 256-thread block per row and walks the row three times (mean, variance,
//    normalise) forward and twice backward, with two float atomics per ELEMENT for grad_gamma / grad_beta. Here a warp
//    owns a row and keeps it in registers (a 768-wide row is six float4 per lane): one read and one write of the
//    activations forward, two reads and one write backward; grad_gamma / grad_beta are summed in registers over all rows
//    a warp sees, then in shared memory over the block, and reach global memory as one atomic per column and BLOCK.
//  * GELU: 16-byte accesses; tanh through one exponential, 0.5 * (1 + tanh(u)) = 1 / (1 + exp(-2u)).
//  * AdamW: the reference launches once per parameter tensor (196 launches for a 12-layer GPT-2 small, most of them over a few
//    thousand elements). df_adamw_update_multi walks a caller-built table of tensors in ONE launch, in chunks of 2048
//    elements dealt over a grid sized to the machine.
#include <math.h>

#include <mutex>

#include "df_common.cuh"
#include "sm100_ptx.cuh"

namespace df {
namespace {
using namespace ptx;

constexpr float kLnEps = 1e-5f;           // layernorm.cu:14
constexpr int kRowThreads = 256;          // eight warps, one row each at a time
constexpr uint32_t kAdamChunk = 2048;     // elements of one work unit of the multi-tensor update

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float sum4(const float4 &a) { return (a.x + a.y) + (a.z + a.w); }

// ------------------------------------------------------------------------------------------------ LayerNorm forward
// One warp per row, grid-stride over rows; VPL float4 per lane hold the row (cols <= 128 * VPL, cols % 4 == 0, rows
// 16-byte aligned). Mean and variance in two passes over the registers, as the reference does over memory.
template <int VPL>
__global__ void __launch_bounds__(kRowThreads)
k_layernorm_fwd(const float *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                float *__restrict__ out, float *__restrict__ means, float *__restrict__ rstds, uint32_t rows, uint32_t cols) {
  const uint32_t lane = threadIdx.x & 31u, nvec = cols >> 2;
  const uint32_t warps = gridDim.x * (kRowThreads / 32);
  const float inv_n = 1.0f / (float)cols;
  for (uint32_t row = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * cols);
    float4 v[VPL];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t c = i * 32 + lane;
      v[i] = c < nvec ? __ldcs(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += sum4(v[i]);
    }
    const float mean = warp_sum(s) * inv_n;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if ((uint32_t)(i * 32) + lane < nvec) {
        const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
        q += (a * a + b * b) + (c * c + d * d);
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_n + kLnEps);
    if (lane == 0) {
      if (means) means[row] = mean;
      if (rstds) rstds[row] = rstd;
    }
    float4 *orow = reinterpret_cast<float4 *>(out + (size_t)row * cols);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t c = i * 32 + lane;
      if (c < nvec) {
        const float4 g = gamma ? __ldg(reinterpret_cast<const float4 *>(gamma) + c) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 b = beta ? __ldg(reinterpret_cast<const float4 *>(beta) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 o;
        o.x = (v[i].x - mean) * rstd * g.x + b.x;
        o.y = (v[i].y - mean) * rstd * g.y + b.y;
        o.z = (v[i].z - mean) * rstd * g.z + b.z;
        o.w = (v[i].w - mean) * rstd * g.w + b.w;
        __stcs(orow + c, o);
      }
    }
  }
}

// Any width and alignment: one block per row at a time, the row read three times (the later passes out of L1/L2).
__device__ __forceinline__ float block_sum(float v, float *red) {
  v = warp_sum(v);
  __syncthreads();  // red may still be read from the call before
  if ((threadIdx.x & 31u) == 0u) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for (int w = 0; w < kRowThreads / 32; ++w) t += red[w];
  return t;
}

__global__ void __launch_bounds__(kRowThreads)
k_layernorm_fwd_any(const float *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                    float *__restrict__ out, float *__restrict__ means, float *__restrict__ rstds, uint32_t rows, uint32_t cols) {
  __shared__ float red[kRowThreads / 32];
  const float inv_n = 1.0f / (float)cols;
  for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float *xr = x + (size_t)row * cols;
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += kRowThreads) s += xr[i];
    const float mean = block_sum(s, red) * inv_n;
    float q = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += kRowThreads) {
      const float d = xr[i] - mean;
      q += d * d;
    }
    const float rstd = rsqrtf(block_sum(q, red) * inv_n + kLnEps);
    if (threadIdx.x == 0) {
      if (means) means[row] = mean;
      if (rstds) rstds[row] = rstd;
    }
    float *orow = out + (size_t)row * cols;
    for (uint32_t i = threadIdx.x; i < cols; i += kRowThreads)
      orow[i] = (xr[i] - mean) * rstd * (gamma ? __ldg(gamma + i) : 1.0f) + (beta ? __ldg(beta + i) : 0.0f);
  }
}

// ------------------------------------------------------------------------------------------------ LayerNorm backward
// grad_x[i] = rstd / n * (n * ds_i - sum(ds) - xhat_i * sum(ds * xhat)),  ds = grad_out * gamma   (layernorm.cu:176-182)
// grad_gamma[i] += sum_rows grad_out * xhat,  grad_beta[i] += sum_rows grad_out                   (layernorm.cu:147-148)
// One warp per row, grid-stride; the column sums stay in registers while the warp walks its rows, are added up over
// the block's warps in shared memory (2 * cols floats of dynamic shared memory), and leave with one atomic per column
// and block. cols <= 1024, cols % 4 == 0.
template <int VPL>
__global__ void __launch_bounds__(kRowThreads, VPL <= 6 ? 2 : 1)
k_layernorm_bwd(const float *__restrict__ grad_out, const float *__restrict__ x, const float *__restrict__ gamma,
                const float *__restrict__ means, const float *__restrict__ rstds, float *__restrict__ grad_x,
                float *__restrict__ grad_gamma, float *__restrict__ grad_beta, uint32_t rows, uint32_t cols) {
  extern __shared__ float col_sums[];  // [cols] grad_gamma partials, [cols] grad_beta partials
  const uint32_t lane = threadIdx.x & 31u, nvec = cols >> 2;
  const uint32_t warps = gridDim.x * (kRowThreads / 32);
  const float n = (float)cols;
  const bool want_cols = grad_gamma != nullptr || grad_beta != nullptr;
  for (uint32_t i = threadIdx.x; i < 2 * cols; i += kRowThreads) col_sums[i] = 0.0f;
  __syncthreads();
  float4 ag[VPL], ab[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) ag[i] = ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t row = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * cols);
    const float4 *dr = reinterpret_cast<const float4 *>(grad_out + (size_t)row * cols);
    const float mean = __ldg(means + row), rstd = __ldg(rstds + row);
    float4 xh[VPL], ds[VPL];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t c = i * 32 + lane;
      if (c < nvec) {
        const float4 xv = __ldcs(xr + c), dv = __ldcs(dr + c);
        // gamma comes out of L1 on every row: keeping it in registers too costs the second resident block
        const float4 g = gamma ? __ldg(reinterpret_cast<const float4 *>(gamma) + c) : make_float4(1.f, 1.f, 1.f, 1.f);
        xh[i] = make_float4((xv.x - mean) * rstd, (xv.y - mean) * rstd, (xv.z - mean) * rstd, (xv.w - mean) * rstd);
        ds[i] = make_float4(dv.x * g.x, dv.y * g.y, dv.z * g.z, dv.w * g.w);
        s1 += sum4(ds[i]);
        s2 += (ds[i].x * xh[i].x + ds[i].y * xh[i].y) + (ds[i].z * xh[i].z + ds[i].w * xh[i].w);
        ag[i].x += dv.x * xh[i].x; ag[i].y += dv.y * xh[i].y; ag[i].z += dv.z * xh[i].z; ag[i].w += dv.w * xh[i].w;
        ab[i].x += dv.x; ab[i].y += dv.y; ab[i].z += dv.z; ab[i].w += dv.w;
      } else {
        xh[i] = ds[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const float sum_ds = warp_sum(s1), sum_dsx = warp_sum(s2), f = rstd / n;
    float4 *gx = reinterpret_cast<float4 *>(grad_x + (size_t)row * cols);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t c = i * 32 + lane;
      if (c < nvec)
        __stcs(gx + c, make_float4(f * (n * ds[i].x - sum_ds - xh[i].x * sum_dsx), f * (n * ds[i].y - sum_ds - xh[i].y * sum_dsx),
                                   f * (n * ds[i].z - sum_ds - xh[i].z * sum_dsx), f * (n * ds[i].w - sum_ds - xh[i].w * sum_dsx)));
    }
  }
  if (!want_cols) return;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const uint32_t c = i * 32 + lane;
    if (c < nvec) {
      float *sg = col_sums + 4 * c, *sb = col_sums + cols + 4 * c;
      atomicAdd(sg + 0, ag[i].x); atomicAdd(sg + 1, ag[i].y); atomicAdd(sg + 2, ag[i].z); atomicAdd(sg + 3, ag[i].w);
      atomicAdd(sb + 0, ab[i].x); atomicAdd(sb + 1, ab[i].y); atomicAdd(sb + 2, ab[i].z); atomicAdd(sb + 3, ab[i].w);
    }
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < cols; i += kRowThreads) {
    if (grad_gamma) atomicAdd(grad_gamma + i, col_sums[i]);
    if (grad_beta) atomicAdd(grad_beta + i, col_sums[cols + i]);
  }
}

// The same backward with the rows staged in shared memory by the copy engine: every warp owns a ring of `stages`
// slots of (x row, grad_out row) and keeps `stages` rows in flight ahead of the one it works on, so the loads in
// flight no longer depend on how many registers and warps an SM holds (the register form above runs at 0.6 of the
// copy peak: 16 warps per SM that each wait for their own row). One block per SM; lane 0 of a warp issues its copies.
// Every wait is bounded: a warp whose row does not arrive raises the device status and the block leaves together.
constexpr uint32_t kStagedSmemBudget = 200 * 1024;
template <int VPL>
__global__ void __launch_bounds__(512, 1)
k_layernorm_bwd_staged(const float *__restrict__ grad_out, const float *__restrict__ x, const float *__restrict__ gamma,
                       const float *__restrict__ means, const float *__restrict__ rstds, float *__restrict__ grad_x,
                       float *__restrict__ grad_gamma, float *__restrict__ grad_beta, uint32_t rows, uint32_t cols, uint32_t stages,
                       unsigned int *status) {
  extern __shared__ __align__(128) uint8_t staged_smem[];
  const uint32_t n_warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, nvec = cols >> 2;
  const uint32_t row_bytes = cols * 4u;
  uint64_t *bars = reinterpret_cast<uint64_t *>(staged_smem);                                  // [n_warps * stages]
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(bars + n_warps * stages);
  uint8_t *ring = staged_smem + ((n_warps * stages * 8u + 16u + 127u) & ~127u);  // [n_warps][stages][2][cols]
  uint8_t *my_ring = ring + (size_t)warp * stages * 2u * row_bytes;
  uint64_t *my_bars = bars + warp * stages;
  if (lane == 0)
    for (uint32_t st = 0; st < stages; ++st) mbar_init(smem_u32(my_bars + st), 1);
  if (threadIdx.x == 0) *abort_flag = 0u;
  mbar_init_fence();
  fence_proxy_async_smem();
  __syncthreads();
  const uint32_t total_warps = gridDim.x * n_warps, w0 = blockIdx.x * n_warps + warp;
  const float n = (float)cols;
  // the copies of this warp's k-th row (row w0 + k * total_warps) into slot `st`
  // Lane `st` also fetches the row's mean and rstd now and hands them to the warp when the slot is consumed: loaded
  // at that point instead, the two scalars (a new 32-byte sector on every row) would put a DRAM round trip in
  // front of every row's arithmetic.
  float slot_mean = 0.0f, slot_rstd = 0.0f;
  auto issue = [&](uint32_t row, uint32_t st) {
    if (row < rows) {
      if (lane == 0) {
        const uint32_t bar = smem_u32(my_bars + st), dst = smem_u32(my_ring + (size_t)st * 2u * row_bytes);
        mbar_arrive_expect_tx(bar, 2u * row_bytes);
        bulk_load(dst, x + (size_t)row * cols, row_bytes, bar);
        bulk_load(dst + row_bytes, grad_out + (size_t)row * cols, row_bytes, bar);
      }
      if (lane == st) {
        slot_mean = __ldg(means + row);
        slot_rstd = __ldg(rstds + row);
      }
    }
  };
  for (uint32_t st = 0; st < stages; ++st) issue(w0 + st * total_warps, st);
  float4 ag[VPL], ab[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) ag[i] = ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  bool ok = true;
  uint32_t st = 0, phase = 0;
  for (uint32_t row = w0; row < rows; row += total_warps) {
    if (!mbar_wait_warp(smem_u32(my_bars + st), phase, abort_flag)) { ok = false; break; }
    const float4 *sx = reinterpret_cast<const float4 *>(my_ring + (size_t)st * 2u * row_bytes), *sd = sx + nvec;
    const float mean = __shfl_sync(0xffffffffu, slot_mean, (int)st), rstd = __shfl_sync(0xffffffffu, slot_rstd, (int)st);
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t c = i * 32 + lane;
      if (c < nvec) {
        const float4 xv = sx[c], dv = sd[c];
        const float4 g = gamma ? __ldg(reinterpret_cast<const float4 *>(gamma) + c) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 xh = make_float4((xv.x - mean) * rstd, (xv.y - mean) * rstd, (xv.z - mean) * rstd, (xv.w - mean) * rstd);
        const float4 ds = make_float4(dv.x * g.x, dv.y * g.y, dv.z * g.z, dv.w * g.w);
        s1 += sum4(ds);
        s2 += (ds.x * xh.x + ds.y * xh.y) + (ds.z * xh.z + ds.w * xh.w);
        ag[i].x += dv.x * xh.x; ag[i].y += dv.y * xh.y; ag[i].z += dv.z * xh.z; ag[i].w += dv.w * xh.w;
        ab[i].x += dv.x; ab[i].y += dv.y; ab[i].z += dv.z; ab[i].w += dv.w;
      }
    }
    const float sum_ds = warp_sum(s1), sum_dsx = warp_sum(s2), f = rstd / n;
    float4 *gx = reinterpret_cast<float4 *>(grad_x + (size_t)row * cols);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t c = i * 32 + lane;
      if (c < nvec) {
        const float4 xv = sx[c], dv = sd[c];
        const float4 g = gamma ? __ldg(reinterpret_cast<const float4 *>(gamma) + c) : make_float4(1.f, 1.f, 1.f, 1.f);
        float4 o;
        o.x = f * (n * (dv.x * g.x) - sum_ds - (xv.x - mean) * rstd * sum_dsx);
        o.y = f * (n * (dv.y * g.y) - sum_ds - (xv.y - mean) * rstd * sum_dsx);
        o.z = f * (n * (dv.z * g.z) - sum_ds - (xv.z - mean) * rstd * sum_dsx);
        o.w = f * (n * (dv.w * g.w) - sum_ds - (xv.w - mean) * rstd * sum_dsx);
        __stcs(gx + c, o);
      }
    }
    __syncwarp();  // every lane has read the slot before the copy engine refills it
    issue(row + stages * total_warps, st);
    if (++st == stages) {
      st = 0;
      phase ^= 1u;
    }
  }
  if (!ok && lane == 0) {
    // a row never arrived: report it, and give copies still in flight time to land before the block's shared memory goes
    if (status) atomicOr(status, DEV_STATUS_WAIT_EXPIRED);
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) {
    }
  }
  // Column sums over the block: every warp parks its partial sums in its own ring (empty by now: every copy it issued
  // has been consumed), then each thread adds up a few columns over the warps and sends one atomic per column.
  // (Floating-point atomics on shared memory from sixteen warps at once cost a quarter of the kernel's time.)
  const bool want_cols = grad_gamma != nullptr || grad_beta != nullptr;
  float4 *park = reinterpret_cast<float4 *>(my_ring);  // [2][nvec]
  if (want_cols) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t c = i * 32 + lane;
      if (c < nvec) {
        park[c] = ag[i];
        park[nvec + c] = ab[i];
      }
    }
  }
  __syncthreads();
  if (want_cols) {
    const size_t warp_stride = (size_t)stages * 2u * row_bytes / sizeof(float);
    const float *base = reinterpret_cast<const float *>(ring);
    for (uint32_t i = threadIdx.x; i < 2 * cols; i += blockDim.x) {
      float t = 0.0f;
      for (uint32_t w = 0; w < n_warps; ++w) t += base[w * warp_stride + i];
      float *dst = i < cols ? grad_gamma : grad_beta;
      if (dst) atomicAdd(dst + (i < cols ? i : i - cols), t);
    }
  }
}

// Any width and alignment: a block walks its rows; a thread owns the columns t, t + 256, ... and adds its row's
// contribution to grad_gamma / grad_beta in global memory (the reference's form, layernorm.cu:140-149).
__global__ void __launch_bounds__(kRowThreads)
k_layernorm_bwd_any(const float *__restrict__ grad_out, const float *__restrict__ x, const float *__restrict__ gamma,
                    const float *__restrict__ means, const float *__restrict__ rstds, float *__restrict__ grad_x,
                    float *__restrict__ grad_gamma, float *__restrict__ grad_beta, uint32_t rows, uint32_t cols) {
  __shared__ float red[kRowThreads / 32];
  const float n = (float)cols;
  for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float *xr = x + (size_t)row * cols, *dr = grad_out + (size_t)row * cols;
    const float mean = means[row], rstd = rstds[row];
    float s1 = 0.0f, s2 = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += kRowThreads) {
      const float xh = (xr[i] - mean) * rstd, d = dr[i], ds = d * (gamma ? __ldg(gamma + i) : 1.0f);
      s1 += ds;
      s2 += ds * xh;
      if (grad_gamma) atomicAdd(grad_gamma + i, d * xh);
      if (grad_beta) atomicAdd(grad_beta + i, d);
    }
    const float sum_ds = block_sum(s1, red);
    const float sum_dsx = block_sum(s2, red);
    const float f = rstd / n;
    float *gx = grad_x + (size_t)row * cols;
    for (uint32_t i = threadIdx.x; i < cols; i += kRowThreads) {
      const float xh = (xr[i] - mean) * rstd, ds = dr[i] * (gamma ? __ldg(gamma + i) : 1.0f);
      gx[i] = f * (n * ds - sum_ds - xh * sum_dsx);
    }
  }
}

// ------------------------------------------------------------------------------------------------ GELU
// (gelu_value / gelu_slope: df_common.cuh, shared with the projection kernel's epilogue)
__device__ __forceinline__ float gelu_f(float v) { return gelu_value(v); }
__device__ __forceinline__ float gelu_grad_f(float v) { return gelu_slope(v); }

template <bool VEC>
__global__ void __launch_bounds__(256) k_gelu_fwd(const float *__restrict__ x, float *__restrict__ out, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, t0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {
    const uint64_t nv = n >> 2;
    for (uint64_t i = t0; i < nv; i += stride) {
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(x) + i);
      __stcs(reinterpret_cast<float4 *>(out) + i, make_float4(gelu_f(v.x), gelu_f(v.y), gelu_f(v.z), gelu_f(v.w)));
    }
    for (uint64_t i = (nv << 2) + t0; i < n; i += stride) out[i] = gelu_f(x[i]);
  } else {
    for (uint64_t i = t0; i < n; i += stride) out[i] = gelu_f(x[i]);
  }
}

template <bool VEC>
__global__ void __launch_bounds__(256)
k_gelu_bwd(const float *__restrict__ grad_out, const float *__restrict__ x, float *__restrict__ grad_x, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, t0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {
    const uint64_t nv = n >> 2;
    for (uint64_t i = t0; i < nv; i += stride) {
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(x) + i), d = __ldcs(reinterpret_cast<const float4 *>(grad_out) + i);
      __stcs(reinterpret_cast<float4 *>(grad_x) + i,
             make_float4(d.x * gelu_grad_f(v.x), d.y * gelu_grad_f(v.y), d.z * gelu_grad_f(v.z), d.w * gelu_grad_f(v.w)));
    }
    for (uint64_t i = (nv << 2) + t0; i < n; i += stride) grad_x[i] = grad_out[i] * gelu_grad_f(x[i]);
  } else {
    for (uint64_t i = t0; i < n; i += stride) grad_x[i] = grad_out[i] * gelu_grad_f(x[i]);
  }
}

// ------------------------------------------------------------------------------------------------ AdamW
struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bias_correction1, bias_correction2;
};

// One element, in the reference's order of operations (matmul.cu:310-316).
__device__ __forceinline__ void adamw_one(float &p, float &m, float &v, float g, const AdamHyper &h) {
  m = h.beta1 * m + (1.0f - h.beta1) * g;
  v = h.beta2 * v + (1.0f - h.beta2) * (g * g);
  const float m_hat = m / h.bias_correction1;
  const float v_hat = v / h.bias_correction2;
  const float decay_factor = 1.0f - h.lr * h.weight_decay;
  p = p * decay_factor - h.lr * m_hat / (sqrtf(v_hat) + h.eps);
}

// `n` elements starting at the four pointers; the calling threads are `nthreads` wide with index `t`.
__device__ __forceinline__ void adamw_span(float *__restrict__ p, float *__restrict__ m, float *__restrict__ v,
                                           const float *__restrict__ g, uint64_t n, uint64_t t, uint64_t nthreads,
                                           const AdamHyper &h) {
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                     reinterpret_cast<uintptr_t>(g)) & 15u) == 0;
  uint64_t done = 0;
  if (vec) {
    const uint64_t nv = n >> 2;
    for (uint64_t i = t; i < nv; i += nthreads) {
      float4 pp = reinterpret_cast<float4 *>(p)[i], mm = reinterpret_cast<float4 *>(m)[i], vv = reinterpret_cast<float4 *>(v)[i];
      const float4 gg = __ldcs(reinterpret_cast<const float4 *>(g) + i);
      adamw_one(pp.x, mm.x, vv.x, gg.x, h);
      adamw_one(pp.y, mm.y, vv.y, gg.y, h);
      adamw_one(pp.z, mm.z, vv.z, gg.z, h);
      adamw_one(pp.w, mm.w, vv.w, gg.w, h);
      reinterpret_cast<float4 *>(p)[i] = pp;
      reinterpret_cast<float4 *>(m)[i] = mm;
      reinterpret_cast<float4 *>(v)[i] = vv;
    }
    done = nv << 2;
  }
  for (uint64_t i = done + t; i < n; i += nthreads) {
    float pp = p[i], mm = m[i], vv = v[i];
    adamw_one(pp, mm, vv, g[i], h);
    p[i] = pp;
    m[i] = mm;
    v[i] = vv;
  }
}

__global__ void __launch_bounds__(256)
k_adamw(float *__restrict__ p, float *__restrict__ m, float *__restrict__ v, const float *__restrict__ g, uint64_t n, AdamHyper h) {
  adamw_span(p, m, v, g, n, (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, (uint64_t)gridDim.x * blockDim.x, h);
}

// Work unit = kAdamChunk consecutive elements of one tensor; unit u belongs to the tensor t with
// first_chunk[t] <= u < first_chunk[t + 1] (found by bisection over the table, which sits in L1/L2 after the first units).
__global__ void __launch_bounds__(256)
k_adamw_multi(const df_adamw_tensor_t *__restrict__ tensors, uint32_t n_tensors, uint64_t total_chunks, AdamHyper h) {
  for (uint64_t u = blockIdx.x; u < total_chunks; u += gridDim.x) {
    uint32_t lo = 0, hi = n_tensors - 1;
    while (lo < hi) {
      const uint32_t mid = (lo + hi + 1) >> 1;
      if (tensors[mid].first_chunk <= u) lo = mid; else hi = mid - 1;
    }
    const df_adamw_tensor_t t = tensors[lo];
    const uint64_t off = (u - t.first_chunk) * kAdamChunk;
    if (off >= t.n) continue;  // a table whose first_chunk values leave gaps
    const uint64_t len = t.n - off < kAdamChunk ? t.n - off : kAdamChunk;
    adamw_span(t.parameter + off, t.first_moment + off, t.second_moment + off, t.gradient + off, len, threadIdx.x, blockDim.x, h);
  }
}

std::once_flag g_sm_once[64];
int g_sm_count[64];
int sm_count() {
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev)) != DF_OK || dev < 0 || dev >= 64) return 0;
  std::call_once(g_sm_once[dev], [&]() {
    int n = 0;
    g_sm_count[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 0;
  });
  return g_sm_count[dev];
}

// Blocks of a backward LayerNorm kernel that fit on one SM (queried once per kernel; 8 KB of shared memory assumed).
template <typename K>
uint32_t resident_blocks(K kernel, int slot) {
  static std::once_flag once[2];
  static int blocks[2];
  std::call_once(once[slot], [&]() {
    int b = 0;
    blocks[slot] = (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, kernel, kRowThreads, 8192) == cudaSuccess && b > 0) ? b : 1;
  });
  return (uint32_t)blocks[slot];
}

// Lets the staged LayerNorm backward use more than 48 KB of dynamic shared memory (once per device).
bool staged_ready() {
  static std::once_flag once[64];
  static bool ok[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::call_once(once[dev], [&]() {
    ok[dev] = cudaFuncSetAttribute(k_layernorm_bwd_staged<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) == cudaSuccess &&
              cudaFuncSetAttribute(k_layernorm_bwd_staged<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) == cudaSuccess;
  });
  return ok[dev];
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

AdamHyper hyper(float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2) {
  return AdamHyper{lr, beta1, beta2, eps, weight_decay, bc1, bc2};
}

}  // namespace

int layernorm_forward(const float *x, const float *gamma, const float *beta, float *out, float *means, float *rstds,
                      uint32_t rows, uint32_t cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return DF_OK;
  if (!x || !out) return DF_ERR_INVALID_ARG;
  const int n_sm = sm_count();
  if (n_sm <= 0) return DF_ERR_CUDA;
  const bool vec = (cols & 3u) == 0 && aligned16(x) && aligned16(out) && (!gamma || aligned16(gamma)) && (!beta || aligned16(beta));
  const uint32_t row_blocks = (rows + kRowThreads / 32 - 1) / (kRowThreads / 32);
  // the register kernels get one row per warp (a block costs nothing to start, and the hardware deals blocks to SMs
  // as they free up: with a grid sized to the machine and 3.5 rows per warp the last round ran a quarter full)
  const uint32_t cap = vec && cols <= 4096 ? row_blocks : (uint32_t)n_sm * 8u;
  if (vec && cols <= 768) {
    k_layernorm_fwd<6><<<row_blocks < cap ? row_blocks : cap, kRowThreads, 0, s>>>(x, gamma, beta, out, means, rstds, rows, cols);
  } else if (vec && cols <= 1024) {
    k_layernorm_fwd<8><<<row_blocks < cap ? row_blocks : cap, kRowThreads, 0, s>>>(x, gamma, beta, out, means, rstds, rows, cols);
  } else if (vec && cols <= 4096) {
    k_layernorm_fwd<32><<<row_blocks < cap ? row_blocks : cap, kRowThreads, 0, s>>>(x, gamma, beta, out, means, rstds, rows, cols);
  } else {
    k_layernorm_fwd_any<<<rows < cap ? rows : cap, kRowThreads, 0, s>>>(x, gamma, beta, out, means, rstds, rows, cols);
  }
  note_launch();
  return check_cuda(cudaGetLastError());
}

int layernorm_backward(const float *grad_out, const float *x, const float *gamma, const float *means, const float *rstds,
                       float *grad_x, float *grad_gamma, float *grad_beta, uint32_t rows, uint32_t cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return DF_OK;
  if (!grad_out || !x || !means || !rstds || !grad_x) return DF_ERR_INVALID_ARG;
  const int n_sm = sm_count();
  if (n_sm <= 0) return DF_ERR_CUDA;
  const bool vec = (cols & 3u) == 0 && cols <= 1024 && aligned16(grad_out) && aligned16(x) && aligned16(grad_x) &&
                   (!gamma || aligned16(gamma));
  if (vec) {
    // as many blocks as are resident at once (the registers allow one or two per SM): every block ends with one
    // global atomic per column, so more blocks than that would only add atomics
    const uint32_t row_blocks = (rows + kRowThreads / 32 - 1) / (kRowThreads / 32);
    const size_t smem = 2 * (size_t)cols * sizeof(float);
    // Enough rows to fill the machine: the staged form, 16 warps per SM (8 for wide rows) with 2 to 4 rows in flight each
    const uint32_t row_bytes = cols * 4u;
    const uint32_t warps = (kStagedSmemBudget / (16u * 2u * row_bytes) >= 2u) ? 16u : 8u;
    uint32_t stages = kStagedSmemBudget / (warps * 2u * row_bytes);
    stages = stages > 4u ? 4u : stages;
    if (option(DF_OPT_LN_STAGED) != 0 && stages >= 2u && rows >= (uint32_t)n_sm * warps && staged_ready()) {
      const size_t bytes = ((warps * stages * 8u + 16u + 127u) & ~127u) + (size_t)warps * stages * 2u * row_bytes;
      if (cols <= 768)
        k_layernorm_bwd_staged<6><<<n_sm, warps * 32, bytes, s>>>(grad_out, x, gamma, means, rstds, grad_x, grad_gamma, grad_beta, rows,
                                                                  cols, stages, device_status_ptr());
      else
        k_layernorm_bwd_staged<8><<<n_sm, warps * 32, bytes, s>>>(grad_out, x, gamma, means, rstds, grad_x, grad_gamma, grad_beta, rows,
                                                                  cols, stages, device_status_ptr());
      note_launch();
      return check_cuda(cudaGetLastError());
    }
    if (cols <= 768) {
      const uint32_t cap = (uint32_t)n_sm * resident_blocks(k_layernorm_bwd<6>, 0);
      k_layernorm_bwd<6><<<row_blocks < cap ? row_blocks : cap, kRowThreads, smem, s>>>(grad_out, x, gamma, means, rstds, grad_x,
                                                                                      grad_gamma, grad_beta, rows, cols);
    } else {
      const uint32_t cap = (uint32_t)n_sm * resident_blocks(k_layernorm_bwd<8>, 1);
      k_layernorm_bwd<8><<<row_blocks < cap ? row_blocks : cap, kRowThreads, smem, s>>>(grad_out, x, gamma, means, rstds, grad_x,
                                                                                      grad_gamma, grad_beta, rows, cols);
    }
  } else {
    const uint32_t cap = (uint32_t)n_sm * 8u;
    k_layernorm_bwd_any<<<rows < cap ? rows : cap, kRowThreads, 0, s>>>(grad_out, x, gamma, means, rstds, grad_x, grad_gamma,
                                                                        grad_beta, rows, cols);
  }
  note_launch();
  return check_cuda(cudaGetLastError());
}

int gelu_forward(const float *x, float *out, uint64_t n, cudaStream_t s) {
  if (n == 0) return DF_OK;
  if (!x || !out) return DF_ERR_INVALID_ARG;
  const int n_sm = sm_count();
  if (n_sm <= 0) return DF_ERR_CUDA;
  const uint64_t want = (n / 4 + 255) / 256 + 1, cap = (uint64_t)n_sm * 16;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  if (aligned16(x) && aligned16(out)) k_gelu_fwd<true><<<grid, 256, 0, s>>>(x, out, n);
  else k_gelu_fwd<false><<<grid, 256, 0, s>>>(x, out, n);
  note_launch();
  return check_cuda(cudaGetLastError());
}

int gelu_backward(const float *grad_out, const float *x, float *grad_x, uint64_t n, cudaStream_t s) {
  if (n == 0) return DF_OK;
  if (!grad_out || !x || !grad_x) return DF_ERR_INVALID_ARG;
  const int n_sm = sm_count();
  if (n_sm <= 0) return DF_ERR_CUDA;
  const uint64_t want = (n / 4 + 255) / 256 + 1, cap = (uint64_t)n_sm * 16;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  if (aligned16(x) && aligned16(grad_out) && aligned16(grad_x)) k_gelu_bwd<true><<<grid, 256, 0, s>>>(grad_out, x, grad_x, n);
  else k_gelu_bwd<false><<<grid, 256, 0, s>>>(grad_out, x, grad_x, n);
  note_launch();
  return check_cuda(cudaGetLastError());
}

int adamw_update(float *p, float *m, float *v, const float *g, uint64_t n, float lr, float beta1, float beta2, float eps,
                 float weight_decay, float bc1, float bc2, cudaStream_t s) {
  if (n == 0) return DF_OK;
  if (!p || !m || !v || !g || bc1 == 0.0f || bc2 == 0.0f) return DF_ERR_INVALID_ARG;
  const int n_sm = sm_count();
  if (n_sm <= 0) return DF_ERR_CUDA;
  const uint64_t want = (n / 4 + 255) / 256 + 1, cap = (uint64_t)n_sm * 16;
  k_adamw<<<(unsigned)(want < cap ? want : cap), 256, 0, s>>>(p, m, v, g, n, hyper(lr, beta1, beta2, eps, weight_decay, bc1, bc2));
  note_launch();
  return check_cuda(cudaGetLastError());
}

uint64_t adamw_plan(df_adamw_tensor_t *tensors, uint32_t n_tensors) {
  uint64_t chunks = 0;
  for (uint32_t i = 0; i < n_tensors; ++i) {
    tensors[i].first_chunk = chunks;
    chunks += (tensors[i].n + kAdamChunk - 1) / kAdamChunk;
  }
  return chunks;
}

int adamw_update_multi(const df_adamw_tensor_t *tensors_device, uint32_t n_tensors, uint64_t total_chunks, float lr, float beta1,
                       float beta2, float eps, float weight_decay, float bc1, float bc2, cudaStream_t s) {
  if (n_tensors == 0 || total_chunks == 0) return DF_OK;
  if (!tensors_device || bc1 == 0.0f || bc2 == 0.0f) return DF_ERR_INVALID_ARG;
  const int n_sm = sm_count();
  if (n_sm <= 0) return DF_ERR_CUDA;
  const uint64_t cap = (uint64_t)n_sm * 16;
  k_adamw_multi<<<(unsigned)(total_chunks < cap ? total_chunks : cap), 256, 0, s>>>(tensors_device, n_tensors, total_chunks,
                                                                                    hyper(lr, beta1, beta2, eps, weight_decay, bc1, bc2));
  note_launch();
  return check_cuda(cudaGetLastError());
}

}  // namespace df
