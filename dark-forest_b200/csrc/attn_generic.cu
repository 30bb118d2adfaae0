// attn_generic.cu — shape-generic SIMT attention kernels (any S, 1 <= D <= 128, any alignment).
//
// These are the kernels behind every shape the tcgen05 path does not take (odd head sizes,
// unaligned slices, tiny problems such as the S=5,D=4 and S=4,D=3 cases that the reference's
// own unit tests use, darkforest-cuda/src/lib.rs:2606-2628, 2753-2769), plus the HBM-bound
// helper passes (delta pre-pass, partial-result merge, accumulate).
//
// Arithmetic follows the reference definition (attention_fused.cu:41-159 forward,
// :390-516 backward) but not its structure: a block owns 32 query rows (or 32 keys), four
// lanes share a row and split the head dimension, K/V (or Q/dO) tiles are staged in shared
// memory, the forward saves logsumexp, and the backward is split into a dK/dV kernel and a dQ
// kernel that recompute P from logsumexp, so there is no S x S scratch and no atomics: results
// are bit-reproducible run to run.
#include <math.h>

#include "df_common.cuh"

namespace df {

namespace {

constexpr int kRows = 32;      // rows (queries or keys) owned by a block
constexpr int kTile = 32;      // rows staged per shared-memory tile
constexpr int kThreads = 128;  // 32 rows x 4 lanes

__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// Stage `rows` rows of a [*, dm] tensor (head slice of D floats, zero padded to DP) in smem.
// `base` = element offset of the (batch, head) slice in `src`, `total` = elements of the whole tensor (checked builds).
template <int DP>
__device__ __forceinline__ void stage_tile(float *dst, const float *src, size_t base, long long row0,
                                           long long nrows, size_t dm, uint32_t D, size_t total, unsigned int *status) {
  for (int idx = threadIdx.x; idx < kTile * DP; idx += kThreads) {
    const int j = idx / DP, d = idx % DP;
    const long long r = row0 + j;
    dst[idx] = (r < nrows && d < (int)D) ? __ldg(src + DF_IDX(base + (size_t)r * dm + d, total, status)) : 0.0f;
  }
}

// ---------------------------------------------------------------------------------------
// Forward. Optional outputs: out, lse; "stats" outputs: delta = rowsum(dO * O) without
// materialising O (used by the legacy backward when the caller's scratch cannot hold O).
// ---------------------------------------------------------------------------------------
template <int DPT>
__global__ void __launch_bounds__(kThreads) k_generic_fwd(AttnParams p) {
  constexpr int DP = 4 * DPT;
  __shared__ float sK[kTile * DP];
  __shared__ float sV[kTile * DP];
  const int r = threadIdx.x >> 2, qd = threadIdx.x & 3;
  const uint32_t b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const size_t dm = (size_t)p.H * p.D;
  const long long i = (long long)blockIdx.x * kRows + r;
  const bool row_ok = i < (long long)p.Sq;
  const size_t q_base = (size_t)b * p.Sq * dm + (size_t)h * p.D;
  const size_t k_base = (size_t)b * p.Sk * dm + (size_t)h * p.D;
  // element counts of the q-side tensors, the k-side tensors and the row statistics (used by checked builds only)
  const size_t n_q = (size_t)p.B * p.Sq * dm, n_k = (size_t)p.B * p.Sk * dm, n_s = (size_t)p.B * p.H * p.Sq;
  (void)n_q; (void)n_k; (void)n_s;

  float qreg[DPT], acc[DPT];
#pragma unroll
  for (int t = 0; t < DPT; ++t) {
    const int d = qd + 4 * t;
    qreg[t] = (row_ok && d < (int)p.D) ? __ldg(p.q + DF_IDX(q_base + (size_t)i * dm + d, n_q, p.status)) : 0.0f;
    acc[t] = 0.0f;
  }
  long long last_row = (long long)(blockIdx.x + 1) * kRows;
  if (last_row > (long long)p.Sq) last_row = p.Sq;
  last_row -= 1;
  long long kmax_block = p.causal ? last_row + p.shift + 1 : (long long)p.Sk;
  if (kmax_block > (long long)p.Sk) kmax_block = p.Sk;
  long long my_kmax = p.causal ? i + p.shift + 1 : (long long)p.Sk;
  if (my_kmax > (long long)p.Sk) my_kmax = p.Sk;
  if (!row_ok) my_kmax = 0;

  float m = -INFINITY, l = 0.0f;
  for (long long k0 = 0; k0 < kmax_block; k0 += kTile) {
    __syncthreads();
    stage_tile<DP>(sK, p.k, k_base, k0, p.Sk, dm, p.D, n_k, p.status);
    stage_tile<DP>(sV, p.v, k_base, k0, p.Sk, dm, p.D, n_k, p.status);
    __syncthreads();
    const int jn = (int)((kmax_block - k0) < kTile ? (kmax_block - k0) : kTile);
    for (int j = 0; j < jn; ++j) {
      float part = 0.0f;
#pragma unroll
      for (int t = 0; t < DPT; ++t) part = fmaf(qreg[t], sK[j * DP + qd + 4 * t], part);
      const float s = quad_sum(part) * p.scale;
      if (k0 + j < my_kmax) {
        const float mn = fmaxf(m, s);
        const float alpha = expf(m - mn);  // m = -inf on the first visible key gives 0
        const float pe = expf(s - mn);
        l = fmaf(l, alpha, pe);
        m = mn;
#pragma unroll
        for (int t = 0; t < DPT; ++t) acc[t] = fmaf(pe, sV[j * DP + qd + 4 * t], acc[t] * alpha);
      }
    }
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;  // reference guard, attention_fused.cu:104
  float dpart = 0.0f;
#pragma unroll
  for (int t = 0; t < DPT; ++t) {
    const int d = qd + 4 * t;
    const float o = acc[t] * inv;
    if (row_ok && d < (int)p.D) {
      if (p.out) p.out[DF_IDX(q_base + (size_t)i * dm + d, n_q, p.status)] = o;
      if (p.delta) dpart = fmaf(o, __ldg(p.d_out + DF_IDX(q_base + (size_t)i * dm + d, n_q, p.status)), dpart);
    }
  }
  dpart = quad_sum(dpart);
  if (row_ok && qd == 0) {
    const size_t si = DF_IDX(((size_t)b * p.H + h) * p.Sq + (size_t)i, n_s, p.status);
    if (p.lse) p.lse[si] = l > 0.0f ? m + logf(l) : -INFINITY;
    if (p.delta) p.delta[si] = dpart;
  }
}

// ---------------------------------------------------------------------------------------
// Backward part 1: a block owns 32 keys and walks the query rows that can see them.
//   P = exp(scale*QK^T - lse); dP = dO V^T; dS = P*(dP - delta); dV = P^T dO; dK = scale*dS^T Q
// ---------------------------------------------------------------------------------------
template <int DPT>
__global__ void __launch_bounds__(kThreads) k_generic_bwd_dkdv(AttnParams p) {
  constexpr int DP = 4 * DPT;
  __shared__ float sQ[kTile * DP];
  __shared__ float sG[kTile * DP];
  __shared__ float sLse[kTile], sDelta[kTile];
  const int r = threadIdx.x >> 2, qd = threadIdx.x & 3;
  const uint32_t b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const size_t dm = (size_t)p.H * p.D;
  const long long key0 = (long long)blockIdx.x * kRows;
  const long long kj = key0 + r;
  const bool key_ok = kj < (long long)p.Sk;
  const size_t q_base = (size_t)b * p.Sq * dm + (size_t)h * p.D;
  const size_t k_base = (size_t)b * p.Sk * dm + (size_t)h * p.D;
  const size_t s_base = ((size_t)b * p.H + h) * p.Sq;
  const size_t n_q = (size_t)p.B * p.Sq * dm, n_k = (size_t)p.B * p.Sk * dm, n_s = (size_t)p.B * p.H * p.Sq;
  (void)n_q; (void)n_k; (void)n_s;

  float kreg[DPT], vreg[DPT], dk[DPT], dv[DPT];
#pragma unroll
  for (int t = 0; t < DPT; ++t) {
    const int d = qd + 4 * t;
    const bool ok = key_ok && d < (int)p.D;
    kreg[t] = ok ? __ldg(p.k + DF_IDX(k_base + (size_t)kj * dm + d, n_k, p.status)) : 0.0f;
    vreg[t] = ok ? __ldg(p.v + DF_IDX(k_base + (size_t)kj * dm + d, n_k, p.status)) : 0.0f;
    dk[t] = 0.0f;
    dv[t] = 0.0f;
  }
  // first query row that can see any key of this block: i >= key0 - shift
  long long i_begin = p.causal ? key0 - p.shift : 0;
  if (i_begin < 0) i_begin = 0;
  i_begin = (i_begin / kTile) * kTile;
  for (long long i0 = i_begin; i0 < (long long)p.Sq; i0 += kTile) {
    __syncthreads();
    stage_tile<DP>(sQ, p.q, q_base, i0, p.Sq, dm, p.D, n_q, p.status);
    stage_tile<DP>(sG, p.d_out, q_base, i0, p.Sq, dm, p.D, n_q, p.status);
    if (threadIdx.x < kTile) {
      const long long i = i0 + threadIdx.x;
      sLse[threadIdx.x] = i < (long long)p.Sq ? __ldg(p.lse_in + DF_IDX(s_base + i, n_s, p.status)) : INFINITY;
      sDelta[threadIdx.x] = i < (long long)p.Sq ? __ldg(p.delta_in + DF_IDX(s_base + i, n_s, p.status)) : 0.0f;
    }
    __syncthreads();
    const int in = (int)(((long long)p.Sq - i0) < kTile ? ((long long)p.Sq - i0) : kTile);
    for (int ii = 0; ii < in; ++ii) {
      float ps = 0.0f, pd = 0.0f;
#pragma unroll
      for (int t = 0; t < DPT; ++t) {
        ps = fmaf(sQ[ii * DP + qd + 4 * t], kreg[t], ps);
        pd = fmaf(sG[ii * DP + qd + 4 * t], vreg[t], pd);
      }
      const float s = quad_sum(ps) * p.scale;
      const float dp = quad_sum(pd);
      const bool vis = key_ok && (!p.causal || kj <= i0 + ii + p.shift);
      const float lse_i = sLse[ii];
      const float pr = (vis && lse_i != -INFINITY) ? expf(s - lse_i) : 0.0f;
      const float ds = pr * (dp - sDelta[ii]);
#pragma unroll
      for (int t = 0; t < DPT; ++t) {
        dv[t] = fmaf(pr, sG[ii * DP + qd + 4 * t], dv[t]);
        dk[t] = fmaf(ds, sQ[ii * DP + qd + 4 * t], dk[t]);
      }
    }
  }
  if (key_ok) {
#pragma unroll
    for (int t = 0; t < DPT; ++t) {
      const int d = qd + 4 * t;
      if (d < (int)p.D) {
        p.d_k[DF_IDX(k_base + (size_t)kj * dm + d, n_k, p.status)] = dk[t] * p.scale;
        p.d_v[DF_IDX(k_base + (size_t)kj * dm + d, n_k, p.status)] = dv[t];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Backward part 2: a block owns 32 query rows: dQ = scale * dS K.
// ---------------------------------------------------------------------------------------
template <int DPT>
__global__ void __launch_bounds__(kThreads) k_generic_bwd_dq(AttnParams p) {
  constexpr int DP = 4 * DPT;
  __shared__ float sK[kTile * DP];
  __shared__ float sV[kTile * DP];
  const int r = threadIdx.x >> 2, qd = threadIdx.x & 3;
  const uint32_t b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const size_t dm = (size_t)p.H * p.D;
  const long long i = (long long)blockIdx.x * kRows + r;
  const bool row_ok = i < (long long)p.Sq;
  const size_t q_base = (size_t)b * p.Sq * dm + (size_t)h * p.D;
  const size_t k_base = (size_t)b * p.Sk * dm + (size_t)h * p.D;
  const size_t s_base = ((size_t)b * p.H + h) * p.Sq;
  const size_t n_q = (size_t)p.B * p.Sq * dm, n_k = (size_t)p.B * p.Sk * dm, n_s = (size_t)p.B * p.H * p.Sq;
  (void)n_q; (void)n_k; (void)n_s;

  float qreg[DPT], greg[DPT], dq[DPT];
#pragma unroll
  for (int t = 0; t < DPT; ++t) {
    const int d = qd + 4 * t;
    const bool ok = row_ok && d < (int)p.D;
    qreg[t] = ok ? __ldg(p.q + DF_IDX(q_base + (size_t)i * dm + d, n_q, p.status)) : 0.0f;
    greg[t] = ok ? __ldg(p.d_out + DF_IDX(q_base + (size_t)i * dm + d, n_q, p.status)) : 0.0f;
    dq[t] = 0.0f;
  }
  const float lse_i = row_ok ? __ldg(p.lse_in + DF_IDX(s_base + i, n_s, p.status)) : -INFINITY;
  const float delta_i = row_ok ? __ldg(p.delta_in + DF_IDX(s_base + i, n_s, p.status)) : 0.0f;
  long long last_row = (long long)(blockIdx.x + 1) * kRows;
  if (last_row > (long long)p.Sq) last_row = p.Sq;
  last_row -= 1;
  long long kmax_block = p.causal ? last_row + p.shift + 1 : (long long)p.Sk;
  if (kmax_block > (long long)p.Sk) kmax_block = p.Sk;
  long long my_kmax = p.causal ? i + p.shift + 1 : (long long)p.Sk;
  if (my_kmax > (long long)p.Sk) my_kmax = p.Sk;
  if (!row_ok || lse_i == -INFINITY) my_kmax = 0;

  for (long long k0 = 0; k0 < kmax_block; k0 += kTile) {
    __syncthreads();
    stage_tile<DP>(sK, p.k, k_base, k0, p.Sk, dm, p.D, n_k, p.status);
    stage_tile<DP>(sV, p.v, k_base, k0, p.Sk, dm, p.D, n_k, p.status);
    __syncthreads();
    const int jn = (int)((kmax_block - k0) < kTile ? (kmax_block - k0) : kTile);
    for (int j = 0; j < jn; ++j) {
      float ps = 0.0f, pd = 0.0f;
#pragma unroll
      for (int t = 0; t < DPT; ++t) {
        ps = fmaf(qreg[t], sK[j * DP + qd + 4 * t], ps);
        pd = fmaf(greg[t], sV[j * DP + qd + 4 * t], pd);
      }
      const float s = quad_sum(ps) * p.scale;
      const float dp = quad_sum(pd);
      const float pr = (k0 + j < my_kmax) ? expf(s - lse_i) : 0.0f;
      const float ds = pr * (dp - delta_i);
#pragma unroll
      for (int t = 0; t < DPT; ++t) dq[t] = fmaf(ds, sK[j * DP + qd + 4 * t], dq[t]);
    }
  }
  if (row_ok) {
#pragma unroll
    for (int t = 0; t < DPT; ++t) {
      const int d = qd + 4 * t;
      if (d < (int)p.D) p.d_q[DF_IDX(q_base + (size_t)i * dm + d, n_q, p.status)] = dq[t] * p.scale;
    }
  }
}

// ---------------------------------------------------------------------------------------
// delta pre-pass, HBM-bound: delta[b][h][i] = sum_d dO[b][i][h][d] * O[b][i][h][d].
// A block streams 32 consecutive rows (a contiguous 32*H*D chunk of both tensors) with 16-byte
// loads, LPS = D/4 lanes cooperate on one (row, head) segment, the 32*H sums are transposed
// through shared memory so the [B][H][S] output is written in full 128-byte lines.
// Algorithmic bytes: 2*B*S*H*D*4 read + B*H*S*4 written.
// ---------------------------------------------------------------------------------------
template <int LPS>
__global__ void __launch_bounds__(256) k_delta_vec(const float4 *__restrict__ o,
                                                   const float4 *__restrict__ g,
                                                   float *__restrict__ delta, uint32_t H,
                                                   uint32_t S, uint32_t tiles_per_batch, uint32_t R) {
  extern __shared__ float s_sum[];  // [H][R], R = rows per block (32, or 8 when the grid would be too small)
  const uint32_t b = blockIdx.x / tiles_per_batch;
  const uint32_t i0 = (blockIdx.x % tiles_per_batch) * R;
  const uint32_t rows = (S - i0) < R ? (S - i0) : R;
  const uint32_t nseg = rows * H;  // segments in this chunk, index = ii*H + h
  const size_t chunk = ((size_t)b * S + i0) * H * LPS;  // in float4 units
  const uint32_t grp = threadIdx.x / LPS, lane = threadIdx.x % LPS;
  constexpr uint32_t kGroups = 256 / LPS;
  for (uint32_t sg0 = 0; sg0 < nseg; sg0 += kGroups * 4) {
    float acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t sg = sg0 + u * kGroups + grp;
      acc[u] = 0.0f;
      if (sg < nseg) {
        const float4 a = __ldg(o + chunk + (size_t)sg * LPS + lane);
        const float4 c = __ldg(g + chunk + (size_t)sg * LPS + lane);
        acc[u] = a.x * c.x + a.y * c.y + a.z * c.z + a.w * c.w;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int off = LPS / 2; off > 0; off >>= 1) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], off);
      const uint32_t sg = sg0 + u * kGroups + grp;
      if (lane == 0 && sg < nseg) s_sum[(sg % H) * R + sg / H] = acc[u];
    }
  }
  __syncthreads();
  for (uint32_t idx = threadIdx.x; idx < R * H; idx += 256u) {
    const uint32_t h = idx / R, ii = idx % R;
    if (ii < rows) delta[((size_t)b * H + h) * S + i0 + ii] = s_sum[idx];
  }
}

// Any D / alignment: one thread per (b, h, i).
__global__ void k_delta_scalar(const float *__restrict__ o, const float *__restrict__ g,
                               float *__restrict__ delta, uint32_t B, uint32_t H, uint32_t S,
                               uint32_t D) {
  const size_t n = (size_t)B * H * S;
  for (size_t u = blockIdx.x * (size_t)blockDim.x + threadIdx.x; u < n;
       u += (size_t)gridDim.x * blockDim.x) {
    const size_t i = u % S, h = (u / S) % H, b = (u / S) / H;
    const size_t off = ((b * S + i) * H + h) * D;
    float s = 0.0f;
    for (uint32_t d = 0; d < D; ++d) s = fmaf(__ldg(o + off + d), __ldg(g + off + d), s);
    delta[u] = s;
  }
}

// Partial-result merge (ring step): one thread per (b, i, h, d); weights recomputed per element.
__global__ void k_merge_partials(float *__restrict__ o_a, float *__restrict__ lse_a,
                                 const float *__restrict__ o_b, const float *__restrict__ lse_b,
                                 uint32_t B, uint32_t H, uint32_t S, uint32_t D) {
  const size_t n = (size_t)B * S * H * D;
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n;
       e += (size_t)gridDim.x * blockDim.x) {
    const size_t d = e % D, h = (e / D) % H, i = (e / ((size_t)D * H)) % S,
                 b = e / ((size_t)D * H * S);
    const size_t si = (b * H + h) * S + i;
    const float la = lse_a[si], lb = __ldg(lse_b + si);
    const float mx = fmaxf(la, lb);
    float res = 0.0f;
    if (mx != -INFINITY) {
      const float wa = expf(la - mx), wb = expf(lb - mx);
      res = (wa * o_a[e] + wb * __ldg(o_b + e)) / (wa + wb);
    }
    o_a[e] = res;
  }
}

// Second pass of the merge: the statistics themselves (kept separate so that every element
// thread of the first pass reads the un-merged lse_a).
__global__ void k_merge_lse(float *__restrict__ lse_a, const float *__restrict__ lse_b, size_t n) {
  for (size_t u = blockIdx.x * (size_t)blockDim.x + threadIdx.x; u < n;
       u += (size_t)gridDim.x * blockDim.x) {
    const float la = lse_a[u], lb = __ldg(lse_b + u);
    const float mx = fmaxf(la, lb);
    if (mx != -INFINITY) lse_a[u] = mx + logf(expf(la - mx) + expf(lb - mx));
  }
}

__global__ void k_accumulate(float *__restrict__ dst, const float *__restrict__ src, size_t n) {
  for (size_t u = blockIdx.x * (size_t)blockDim.x + threadIdx.x; u < n;
       u += (size_t)gridDim.x * blockDim.x)
    dst[u] += __ldg(src + u);
}

inline int grid_1d(size_t n, int threads) {
  size_t blocks = (n + threads - 1) / threads;
  const size_t cap = 148 * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

// checked builds hand the kernels the device status word their index checks report to
static inline AttnParams with_status(const AttnParams &p) {
  AttnParams q = p;
#ifdef DF_BOUNDS_CHECK
  q.status = device_status_ptr();
#endif
  return q;
}
#define DF_LAUNCH_BY_D(KERNEL, GRID, P, STREAM)                                               \
  do {                                                                                        \
    const AttnParams df_lp = with_status(P);                                                  \
    if (df_lp.D <= 16) KERNEL<4><<<(GRID), kThreads, 0, (STREAM)>>>(df_lp);                   \
    else if (df_lp.D <= 64) KERNEL<16><<<(GRID), kThreads, 0, (STREAM)>>>(df_lp);             \
    else KERNEL<32><<<(GRID), kThreads, 0, (STREAM)>>>(df_lp);                                \
  } while (0)

int generic_forward(const AttnParams &p, cudaStream_t s) {
  if (p.Sq == 0 || p.B == 0 || p.H == 0) return DF_OK;
  if ((uint64_t)p.B * p.H > 65535u) return DF_ERR_UNSUPPORTED;  // (batch, head) is the grid's y dimension
  dim3 grid((p.Sq + kRows - 1) / kRows, p.B * p.H);
  DF_LAUNCH_BY_D(k_generic_fwd, grid, p, s);
  note_launch();
  return check_cuda(cudaGetLastError());
}

int generic_backward_dkdv(const AttnParams &p, cudaStream_t s) {
  if (p.Sk == 0 || p.B == 0 || p.H == 0) return DF_OK;
  if ((uint64_t)p.B * p.H > 65535u) return DF_ERR_UNSUPPORTED;  // (batch, head) is the grid's y dimension
  dim3 grid((p.Sk + kRows - 1) / kRows, p.B * p.H);
  DF_LAUNCH_BY_D(k_generic_bwd_dkdv, grid, p, s);
  note_launch();
  return check_cuda(cudaGetLastError());
}

int generic_backward_dq(const AttnParams &p, cudaStream_t s) {
  if (p.Sq == 0 || p.B == 0 || p.H == 0) return DF_OK;
  if ((uint64_t)p.B * p.H > 65535u) return DF_ERR_UNSUPPORTED;  // (batch, head) is the grid's y dimension
  dim3 grid((p.Sq + kRows - 1) / kRows, p.B * p.H);
  DF_LAUNCH_BY_D(k_generic_bwd_dq, grid, p, s);
  note_launch();
  return check_cuda(cudaGetLastError());
}

int delta_prepass(const AttnParams &p, cudaStream_t s) {
  if (p.Sq == 0 || p.B == 0 || p.H == 0) return DF_OK;
  const uint32_t D = p.D, H = p.H, S = p.Sq;
  const bool pow2 = (D & (D - 1)) == 0 && D >= 4;
  const bool aligned = ((reinterpret_cast<uintptr_t>(p.o_in) | reinterpret_cast<uintptr_t>(p.d_out)) & 15u) == 0;
  if (pow2 && aligned && H <= 256) {
    // 32 rows per block stream best on large inputs; small inputs get 8 rows so that the grid covers the GPU
    const uint32_t R = ((uint64_t)p.B * ((S + 31) / 32) < 148u * 8u) ? 8u : 32u;
    const uint32_t tiles = (S + R - 1) / R;
    const dim3 grid(p.B * tiles);
    const size_t smem = (size_t)H * R * sizeof(float);
    const float4 *o4 = reinterpret_cast<const float4 *>(p.o_in);
    const float4 *g4 = reinterpret_cast<const float4 *>(p.d_out);
    switch (D / 4) {
      case 1: k_delta_vec<1><<<grid, 256, smem, s>>>(o4, g4, p.delta, H, S, tiles, R); break;
      case 2: k_delta_vec<2><<<grid, 256, smem, s>>>(o4, g4, p.delta, H, S, tiles, R); break;
      case 4: k_delta_vec<4><<<grid, 256, smem, s>>>(o4, g4, p.delta, H, S, tiles, R); break;
      case 8: k_delta_vec<8><<<grid, 256, smem, s>>>(o4, g4, p.delta, H, S, tiles, R); break;
      case 16: k_delta_vec<16><<<grid, 256, smem, s>>>(o4, g4, p.delta, H, S, tiles, R); break;
      default: k_delta_vec<32><<<grid, 256, smem, s>>>(o4, g4, p.delta, H, S, tiles, R); break;
    }
  } else {
    const size_t n = (size_t)p.B * H * S;
    k_delta_scalar<<<grid_1d(n, 256), 256, 0, s>>>(p.o_in, p.d_out, p.delta, p.B, H, S, D);
  }
  note_launch();
  return check_cuda(cudaGetLastError());
}

int merge_partials(float *o_a, float *lse_a, const float *o_b, const float *lse_b, uint32_t B,
                   uint32_t H, uint32_t S, uint32_t D, cudaStream_t s) {
  const size_t n = (size_t)B * S * H * D;
  if (n == 0) return DF_OK;
  k_merge_partials<<<grid_1d(n, 256), 256, 0, s>>>(o_a, lse_a, o_b, lse_b, B, H, S, D);
  k_merge_lse<<<grid_1d((size_t)B * H * S, 256), 256, 0, s>>>(lse_a, lse_b, (size_t)B * H * S);
  note_launch(2);
  return check_cuda(cudaGetLastError());
}

int accumulate(float *dst, const float *src, uint64_t n, cudaStream_t s) {
  if (n == 0) return DF_OK;
  k_accumulate<<<grid_1d(n, 256), 256, 0, s>>>(dst, src, (size_t)n);
  note_launch();
  return check_cuda(cudaGetLastError());
}

}  // namespace df
