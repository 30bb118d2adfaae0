// attn_decode.cu — one-token (decode) attention over a KV cache for B200 (sm_100a).
//
// Replaces kernel_fused_mha_decode_kv, its split-K form with kernel_fused_mha_decode_kv_reduce,
// and the paged / paged split-K / paged bf16 forms
// (darkforest-cuda/kernels/attention_fused.cu:551-626, 635-788, 796-1090): per head
//   out = softmax(scale * q K^T) V   over the first cur_seq_len tokens of the cache.
// The reference runs one warp per head (grid = n_heads), i.e. a dozen warps on the whole GPU.
// This path is pure HBM streaming (2 * T * H * D elements read once), so here the tokens of every
// head are always split over many CTAs:
//   * each CTA takes a contiguous range of tokens of one head; its half-warps (16, or 32 in the cluster form) stride over the
//     tokens (16 lanes x 16 bytes cover 64 dims of a K or V row, two such slots for 128 dims), keep
//     an online softmax state each, and merge the 16 states through shared memory;
//   * entry points WITHOUT scratch buffers launch clusters of 8 CTAs per head: the eight partial
//     states are merged by the cluster's first CTA through distributed shared memory;
//   * the split-K entry points write one partial state (m, l, o[D]) per CTA into the caller's
//     partial buffers (never more chunks than the caller's ceil(T / chunk_size)) and a second,
//     tiny kernel merges them — the same max / exp rescale as the reference's reduce kernel.
// Paged caches resolve the physical page of a token through the int32 block table; the bf16 pool
// variant converts on load. Arithmetic is fp32 throughout (exp2 with the scale folded in).
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <math.h>

#include "df_common.cuh"

namespace cg = cooperative_groups;

namespace df {
namespace {

// threads per CTA: 256 in the split form (several CTAs per SM), 512 in the cluster form, where only
// 8 CTAs per head exist and each must keep more loads in flight
__host__ __device__ constexpr int threads_of(int mode) { return mode == 0 ? 512 : 256; }
constexpr int kCluster = 8;         // CTAs per head in the scratch-free form (portable cluster size)
constexpr float kLog2e = 1.4426950408889634f;

struct DecParams {
  const float *q;
  const void *k, *v;              // fp32 or bf16 rows of n_heads * d_head elements
  const int32_t *block_table;     // nullptr: contiguous cache
  float *out;
  float *pm, *pl, *po;            // partial states (split form only)
  uint32_t H, T, D, page_size;
  uint32_t chunk;                 // tokens per CTA
  uint32_t n_chunks;
  float scale_log2;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 4 consecutive elements of a cache row as floats; `e` is the element offset within the tensor
template <bool BF16>
__device__ __forceinline__ float4 load4(const void *base, size_t e) {
  if (BF16) {
    const uint2 r = __ldg(reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(base) + e));
    return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                       __uint_as_float(r.y & 0xffff0000u));
  }
  return __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(base) + e));
}
template <bool BF16>
__device__ __forceinline__ float load1(const void *base, size_t e) {
  if (BF16) return __uint_as_float((uint32_t)__ldg(static_cast<const uint16_t *>(base) + e) << 16);
  return __ldg(static_cast<const float *>(base) + e);
}

// One CTA: tokens [chunk_idx * chunk, ...) of head h. VEC = 4: d_head % 4 == 0 and 16-byte (bf16:
// 8-byte) aligned rows, lane i of a half-warp owns dims 4i..4i+3 (+64 for the second slot);
// VEC = 1: any d_head <= 128 and alignment, lane i owns dims i, i+16, ...
// SLOTS: register slots per lane (VEC = 4: 1 for d_head <= 64, else 2; VEC = 1: 8). TOK: tokens a
// half-warp fetches per round; with one slot four tokens fit the registers that two tokens of
// two slots take, which keeps the same number of bytes in flight at d_head = 64 as at 128.
// MODE 0: cluster of kCluster CTAs per head merges through distributed shared memory and writes out;
// MODE 1: one partial state per CTA goes to the partial buffers.
template <int VEC, int SLOTS, int TOK, bool BF16, int MODE>
__global__ void __launch_bounds__(threads_of(MODE)) k_attn_decode(const DecParams p) {
  constexpr int kSlots = SLOTS;
  constexpr int kHalfWarps = threads_of(MODE) / 16;
  __shared__ float s_m[kHalfWarps], s_l[kHalfWarps];
  __shared__ float s_o[kHalfWarps][128];
  __shared__ float s_res[2 + 128];  // this CTA's merged state: m, l, o[D]

  const uint32_t h = blockIdx.y, chunk_idx = blockIdx.x;
  const int hw = threadIdx.x >> 4, l16 = threadIdx.x & 15;
  // The two half-warps of a warp walk different tokens and may leave the loop at different times:
  // every shuffle names only the 16 lanes of its own half-warp.
  const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
  const uint32_t D = p.D;
  const size_t dm = (size_t)p.H * D;
  const uint32_t t_begin = chunk_idx * p.chunk;
  const uint32_t t_end = min(p.T, t_begin + p.chunk);

  // this lane's dims and its part of q
  float qv[kSlots * VEC];
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
#pragma unroll
    for (int x = 0; x < VEC; ++x) {
      const uint32_t d = VEC == 4 ? (uint32_t)(s * 64 + l16 * 4 + x) : (uint32_t)(s * 16 + l16);
      qv[s * VEC + x] = d < D ? __ldg(p.q + (size_t)h * D + d) : 0.0f;
    }
  }
  float m = -INFINITY, l = 0.0f;
  float acc[kSlots * VEC];
#pragma unroll
  for (int i = 0; i < kSlots * VEC; ++i) acc[i] = 0.0f;

  auto row_of = [&](uint32_t t) -> size_t {
    if (p.block_table == nullptr) return (size_t)t;
    return (size_t)__ldg(p.block_table + t / p.page_size) * p.page_size + (t % p.page_size);
  };
  // TOK tokens per round so that 2 * TOK row loads are in flight per half-warp
  for (uint32_t t = t_begin + hw; t < t_end; t += TOK * kHalfWarps) {
    bool has[TOK];
    size_t e[TOK];
#pragma unroll
    for (int u = 0; u < TOK; ++u) {
      const uint32_t tu = t + u * kHalfWarps;
      has[u] = tu < t_end;
      e[u] = row_of(has[u] ? tu : t) * dm + (size_t)h * D;  // a missing token re-reads the first one (unused)
    }
    float kk[TOK][kSlots * VEC], vv[TOK][kSlots * VEC];
#pragma unroll
    for (int u = 0; u < TOK; ++u) {
#pragma unroll
      for (int s = 0; s < kSlots; ++s) {
        if (VEC == 4) {
          const uint32_t d = (uint32_t)(s * 64 + l16 * 4);
          const bool in = d < D;
          const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 a = in ? load4<BF16>(p.k, e[u] + d) : z;
          const float4 c = in ? load4<BF16>(p.v, e[u] + d) : z;
          kk[u][s * 4] = a.x; kk[u][s * 4 + 1] = a.y; kk[u][s * 4 + 2] = a.z; kk[u][s * 4 + 3] = a.w;
          vv[u][s * 4] = c.x; vv[u][s * 4 + 1] = c.y; vv[u][s * 4 + 2] = c.z; vv[u][s * 4 + 3] = c.w;
        } else {
          const uint32_t d = (uint32_t)(s * 16 + l16);
          const bool in = d < D;
          kk[u][s] = in ? load1<BF16>(p.k, e[u] + d) : 0.0f;
          vv[u][s] = in ? load1<BF16>(p.v, e[u] + d) : 0.0f;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < TOK; ++u) {
      if (!has[u]) break;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < kSlots * VEC; ++i) dot = fmaf(qv[i], kk[u][i], dot);
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) dot += __shfl_xor_sync(hmask, dot, o);
      const float s2 = dot * p.scale_log2;
      const float m_new = fmaxf(m, s2);
      const float alpha = ex2(m - m_new);  // m = -inf on the first token: 0
      const float pe = ex2(s2 - m_new);
      l = fmaf(l, alpha, pe);
#pragma unroll
      for (int i = 0; i < kSlots * VEC; ++i) acc[i] = fmaf(pe, vv[u][i], acc[i] * alpha);
      m = m_new;
    }
  }

  // merge the 16 half-warp states of the CTA
  if (l16 == 0) { s_m[hw] = m; s_l[hw] = l; }
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
#pragma unroll
    for (int x = 0; x < VEC; ++x) {
      const uint32_t d = VEC == 4 ? (uint32_t)(s * 64 + l16 * 4 + x) : (uint32_t)(s * 16 + l16);
      if (d < 128) s_o[hw][d] = acc[s * VEC + x];
    }
  }
  __syncthreads();
  float M = -INFINITY, L = 0.0f, O = 0.0f;
  const uint32_t d = threadIdx.x;
  if (d < 128) {
#pragma unroll
    for (int w = 0; w < kHalfWarps; ++w) M = fmaxf(M, s_m[w]);
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kHalfWarps; ++w) {
        const float wgt = ex2(s_m[w] - M);
        L = fmaf(s_l[w], wgt, L);
        O = fmaf(s_o[w][d], wgt, O);
      }
    }
  }
  if (MODE == 1) {
    // one partial state per CTA (m in log2 units); a CTA without tokens contributes m = -inf, l = 0
    const size_t slot = (size_t)h * p.n_chunks + chunk_idx;
    if (d == 0) { p.pm[slot] = M; p.pl[slot] = L; }
    if (d < D) p.po[slot * D + d] = O;
  } else {
    cg::cluster_group cluster = cg::this_cluster();
    if (d == 0) { s_res[0] = M; s_res[1] = L; }
    if (d < 128) s_res[2 + d] = O;
    cluster.sync();
    if (cluster.block_rank() == 0 && d < D) {
      float Mg = -INFINITY;
      for (unsigned r = 0; r < cluster.num_blocks(); ++r) Mg = fmaxf(Mg, cluster.map_shared_rank(s_res, r)[0]);
      float Lg = 0.0f, Og = 0.0f;
      if (Mg > -INFINITY) {
        for (unsigned r = 0; r < cluster.num_blocks(); ++r) {
          const float *rs = cluster.map_shared_rank(s_res, r);
          const float wgt = ex2(rs[0] - Mg);
          Lg = fmaf(rs[1], wgt, Lg);
          Og = fmaf(rs[2 + d], wgt, Og);
        }
      }
      p.out[(size_t)h * D + d] = Lg > 0.0f ? Og / Lg : 0.0f;
    }
    cluster.sync();  // the other CTAs' shared memory must outlive the reads above
  }
}

// Merges the partial states of one head: grid = n_heads, 128 threads. The chunk maxima and sums
// are staged in shared memory with coalesced loads, then thread d accumulates output dim d over the
// chunks with independent, unrolled loads (a plain loop of dependent loads cost 11 us for 25 chunks).
// Launched with programmatic stream serialization: its set-up overlaps the tail of the split kernel,
// and griddepcontrol.wait orders it after that kernel's stores.
constexpr int kMaxChunks = 1024;
__global__ void __launch_bounds__(128) k_attn_decode_reduce(const float *__restrict__ pm, const float *__restrict__ pl,
                                                            const float *__restrict__ po, float *__restrict__ out,
                                                            uint32_t n_chunks, uint32_t D) {
  __shared__ float s_w[kMaxChunks];
  __shared__ float s_red[4];
  const uint32_t h = blockIdx.x, d = threadIdx.x;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  float mx = -INFINITY;
  for (uint32_t c = d; c < n_chunks; c += 128) {
    const float mc = pm[(size_t)h * n_chunks + c];
    s_w[c] = mc;
    mx = fmaxf(mx, mc);
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((d & 31) == 0) s_red[d >> 5] = mx;
  __syncthreads();
  const float M = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  __syncthreads();
  float lsum = 0.0f;
  for (uint32_t c = d; c < n_chunks; c += 128) {
    const float w = M > -INFINITY ? ex2(s_w[c] - M) : 0.0f;
    s_w[c] = w;
    lsum = fmaf(pl[(size_t)h * n_chunks + c], w, lsum);
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
  if ((d & 31) == 0) s_red[d >> 5] = lsum;
  __syncthreads();
  const float L = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
  if (d >= D) return;
  float O = 0.0f;
  const float *po_h = po + (size_t)h * n_chunks * D + d;
#pragma unroll 8
  for (uint32_t c = 0; c < n_chunks; ++c) O = fmaf(po_h[(size_t)c * D], s_w[c], O);
  out[(size_t)h * D + d] = L > 0.0f ? O / L : 0.0f;
}

template <int VEC, int SLOTS, int TOK, bool BF16>
int launch(const DecParams &p, bool split, cudaStream_t s) {
  if (split) {
    k_attn_decode<VEC, SLOTS, TOK, BF16, 1><<<dim3(p.n_chunks, p.H), threads_of(1), 0, s>>>(p);
    note_launch();
    if (check_cuda(cudaGetLastError()) != DF_OK) return DF_ERR_CUDA;
    cudaLaunchConfig_t rc = {};
    rc.gridDim = dim3(p.H);
    rc.blockDim = dim3(128);
    rc.stream = s;
    cudaLaunchAttribute ra[1];
    ra[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    ra[0].val.programmaticStreamSerializationAllowed = 1;
    rc.attrs = ra;
    rc.numAttrs = 1;
    const int st = check_cuda(cudaLaunchKernelEx(&rc, k_attn_decode_reduce, (const float *)p.pm, (const float *)p.pl,
                                                 (const float *)p.po, p.out, p.n_chunks, p.D));
    note_launch();
    return st;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kCluster, p.H);
  cfg.blockDim = dim3(threads_of(0));
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int st = check_cuda(cudaLaunchKernelEx(&cfg, k_attn_decode<VEC, SLOTS, TOK, BF16, 0>, p));
  note_launch();
  return st;
}

}  // namespace

// Decode dispatch. partial_* may be null (scratch-free cluster form); otherwise they hold at least
// n_heads * max_chunks states, and the split form is used when it pays (more than one chunk).
int decode_dispatch(const float *q, const void *k, const void *v, const int32_t *block_table, float *out,
                    float *partial_m, float *partial_l, float *partial_o, uint32_t max_chunks, uint32_t H,
                    uint32_t T, uint32_t D, float scale, uint32_t page_size, bool kv_bf16, cudaStream_t s) {
  DecParams p;
  p.q = q; p.k = k; p.v = v; p.block_table = block_table; p.out = out;
  p.pm = partial_m; p.pl = partial_l; p.po = partial_o;
  p.H = H; p.T = T; p.D = D; p.page_size = page_size ? page_size : 1;
  p.scale_log2 = scale * kLog2e;
  bool split = partial_m && partial_l && partial_o && max_chunks > 1;
  // Below about 50 MB of K and V the single cluster launch is faster than split + reduce
  // (measured on B200 at H=12, D=64: 14 vs 20 us at T=4096, 54 vs 44 us at T=32768).
  if ((uint64_t)T * H * D * (kv_bf16 ? 2 : 4) * 2 < (48ull << 20)) split = false;
  if (split) {
    // enough CTAs to fill the GPU about twice, at least 64 tokens each, never more than the caller sized for
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    uint32_t want = (uint32_t)((2 * n_sm + (int)H - 1) / (int)H);
    const uint32_t by_len = (T + 63) / 64;
    if (want > by_len) want = by_len;
    if (want > max_chunks) want = max_chunks;
    if (want > (uint32_t)kMaxChunks) want = kMaxChunks;
    if (want < 2) split = false;
    else {
      p.chunk = (T + want - 1) / want;
      p.n_chunks = (T + p.chunk - 1) / p.chunk;
    }
  }
  if (!split) {
    p.chunk = (T + kCluster - 1) / kCluster;
    if (p.chunk == 0) p.chunk = 1;
    p.n_chunks = kCluster;
  }
  const uintptr_t bits = reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v);
  const bool vec = (D % 4 == 0) && (bits % (kv_bf16 ? 8 : 16) == 0);
  if (kv_bf16) {
    if (!vec) return launch<1, 8, 2, true>(p, split, s);
    return D <= 64 ? launch<4, 1, 4, true>(p, split, s) : launch<4, 2, 2, true>(p, split, s);
  }
  if (!vec) return launch<1, 8, 2, false>(p, split, s);
  return D <= 64 ? launch<4, 1, 4, false>(p, split, s) : launch<4, 2, 2, false>(p, split, s);
}

}  // namespace df
