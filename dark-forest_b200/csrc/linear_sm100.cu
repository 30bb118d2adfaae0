// linear_sm100.cu — the projections on either side of the attention op for B200 (sm_100a):
//   out_j[M, N] = X[M, K] W_j[N, K]^T + b_j[N]  (+ residual[M, N])      j = 0 .. n_mats-1
// as ONE persistent tcgen05 kernel. It replaces, per layer of the reference's static GPT-2 graph,
//   * the three Q/K/V projections, each a cublasSgemm plus a bias pass
//     (darkforest-core/src/engine/static_gpt2.rs:1324-1326 -> darkforest-cuda/src/lib.rs:1138-1201,
//      darkforest-cuda/kernels/elementwise.cu:230-249): one launch writes Q, K and V straight into the
//     [S, H*D] slices the attention kernels read;
//   * the output projection, its bias pass and the first residual add (static_gpt2.rs:1339-1341).
// The CPU engine's definition is cpu_linear (static_gpt2.rs:2717-2733): acc = b[o] + sum_i x[i] w[o, i].
//
// Arithmetic: X and W are rounded to TF32 (nearest even) by the TFLOAT32 tensor maps in flight, products
// accumulate in fp32 in tensor memory, bias and residual are added in fp32 in the epilogue: the same
// arithmetic width as the attention op of the fp32 API.
//
// Structure (one CTA per SM at most, 192 threads):
//   warp 0      TMA producer: a ring of kStages stages, each a 128 x 32 tile of X (16 KB) and a 256 x 32
//               tile of W_j (32 KB), 128-byte swizzle, K-major - both operands are already K-major in
//               global memory (rows of X and rows of W are contiguous along the contraction);
//   warp 1      MMA issuer: 128 x 256 x 8 kind::tf32 SS MMAs (four per stage) into one of two 256-column
//               accumulators in tensor memory, so that the epilogue of tile i overlaps the products of i+1;
//   warps 2-5   epilogue: tensor memory -> registers (+ bias, + residual) -> a 128 x 32 staging slab in
//               shared memory -> bulk tensor store; two slabs alternate.
// Tiles are numbered with the output-feature tile fastest, so CTAs working at the same time share the
// same rows of X through L2 while the W_j (a few MB) stay resident there. Rows beyond M, features beyond N
// and a ragged end of K are handled by the copy engine (zero fill on loads, clipping on stores).
// Every mbarrier wait is bounded (sm100_ptx.cuh); there is no named-barrier or spin wait without a limit.
#include <math.h>
#include <stdio.h>

#include <mutex>

#include "df_common.cuh"
#include "sm100_ptx.cuh"

namespace df {
namespace {

using namespace ptx;

constexpr int TM = 128, TN = 256, TK = 32;
constexpr int kStages = 4;
constexpr int kLinThreads = 192;
constexpr uint32_t kABytes = TM * TK * 4, kBBytes = TN * TK * 4, kStageBytes = kABytes + kBBytes;
constexpr uint32_t kSlabBytes = TM * 32 * 4;                      // one staging slab: 128 rows x 32 floats
constexpr uint32_t kSmemStaging = kStages * kStageBytes;
constexpr uint32_t kSmemBars = kSmemStaging + 2 * kSlabBytes;
constexpr uint32_t kSmemTotal = kSmemBars + 256 + 1024;
constexpr uint32_t kTmemCols = 512;

enum Bar { FULL = 0, EMPTY = FULL + kStages, ACC_FULL = EMPTY + kStages, ACC_EMPTY = ACC_FULL + 2, EPI_A = ACC_EMPTY + 2, EPI_B,
           DRAIN, NUM_BARS };

struct LinParams {
  const float *bias[3];
  const float *residual;
  int gelu;       // 1: one matrix; tmO1 is the map of a second output that receives gelu(x W^T + b)
  int store_pre;  // with gelu: also write the pre-activation through tmO0 (the backward needs it)
  uint32_t M, N, K;
  int n_mats, n_tiles_per_mat, n_tiles_total;  // output-feature tiles per matrix / over all matrices
  long long tiles;
  unsigned int *status;
};

__global__ void __launch_bounds__(kLinThreads, 1)
k_linear_tf32(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW0,
              const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmW2,
              const __grid_constant__ CUtensorMap tmO0, const __grid_constant__ CUtensorMap tmO1,
              const __grid_constant__ CUtensorMap tmO2, const LinParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t a0 = smem_u32(smem);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kSmemBars);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kSmemBars + 192);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + kSmemBars + 196);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto bar = [&](int id) { return smem_u32(&bars[id]); };

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i) mbar_init(bar(i), (i >= ACC_EMPTY && i <= EPI_B) ? 128 : 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW0);
    tma_prefetch_desc(&tmO0);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const int n_kb = (int)((p.K + TK - 1) / TK);

  // tile number -> (row tile, matrix, feature tile); the feature tile runs fastest
  auto decode = [&](long long id, int *m_tile, int *mat, int *n_tile) {
    *m_tile = (int)(id / p.n_tiles_total);
    const int nn = (int)(id % p.n_tiles_total);
    *mat = nn / p.n_tiles_per_mat;
    *n_tile = nn % p.n_tiles_per_mat;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long id = blockIdx.x; ok && id < p.tiles; id += gridDim.x) {
        int m_tile, mat, n_tile;
        decode(id, &m_tile, &mat, &n_tile);
        const CUtensorMap *tw = mat == 0 ? &tmW0 : (mat == 1 ? &tmW1 : &tmW2);
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const uint32_t s = it % kStages, use = it / kStages;
          if (use > 0 && !mbar_wait(bar(EMPTY + s), (use - 1) & 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(bar(FULL + s), kStageBytes);
          tma_load_2d(a0 + s * kStageBytes, &tmX, bar(FULL + s), kb * TK, m_tile * TM);
          tma_load_2d(a0 + s * kStageBytes + kABytes, tw, bar(FULL + s), kb * TK, n_tile * TN);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs this role, warp-uniformly; one elected lane issues the MMA and commit instructions and
    // every wait returns the same answer in all lanes (see elect_one).
    {
      const uint32_t idesc = make_idesc(kFmtTF32, TM, TN, 0, 0);
      uint32_t it = 0, j = 0;
      bool ok = true;
      for (long long id = blockIdx.x; ok && id < p.tiles; id += gridDim.x, ++j) {
        const uint32_t acc = j & 1;
        if (j >= 2 && !mbar_wait_warp(bar(ACC_EMPTY + acc), ((j >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const uint32_t s = it % kStages;
          if (!mbar_wait_warp(bar(FULL + s), (it / kStages) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = a0 + s * kStageBytes, sb = sa + kABytes;
          const uint64_t da = make_smem_desc(sa, 16, 1024, kSwz128), db = make_smem_desc(sb, 16, 1024, kSwz128);
#pragma unroll
          for (int k = 0; k < TK / 8; ++k)
            if (elect_one())
              mma_tf32_ss(tmem + acc * TN, da + (uint64_t)((k * 32) >> 4), db + (uint64_t)((k * 32) >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          commit_elected(bar(EMPTY + s));
        }
        if (ok) commit_elected(bar(ACC_FULL + acc));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (128 threads, one output row each)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const bool issuer = warp == 2 && lane == 0;
    uint32_t j = 0, n_sync_a = 0, n_sync_b = 0, n_store = 0;
    bool ok = true;
    for (long long id = blockIdx.x; ok && id < p.tiles; id += gridDim.x, ++j) {
      int m_tile, mat, n_tile;
      decode(id, &m_tile, &mat, &n_tile);
      const CUtensorMap *to = mat == 0 ? &tmO0 : (mat == 1 ? &tmO1 : &tmO2);
      const float *bias = p.bias[mat];
      const uint32_t acc = j & 1;
      const long long grow = (long long)m_tile * TM + row;
      if (!mbar_wait(bar(ACC_FULL + acc), (j >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      for (int cg = 0; cg < TN / 32; ++cg) {
        const int col0 = n_tile * TN + cg * 32;
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + acc * TN + cg * 32, r);
        tmem_wait_ld();
        if (cg == TN / 32 - 1) {
          // the accumulator has been read completely: the MMA warp may start the tile after next in it
          tc_fence_before_sync();
          mbar_arrive(bar(ACC_EMPTY + acc));
        }
        if (col0 >= (int)p.N) continue;  // a feature tile that ends beyond N (uniform over the CTA)
        float v[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) v[x] = __uint_as_float(r[x]);
        if (bias) {
#pragma unroll
          for (int x4 = 0; x4 < 32; x4 += 4) {
            if (col0 + x4 < (int)p.N) {  // N is a multiple of 4
              const float4 b4 = __ldg(reinterpret_cast<const float4 *>(bias + col0 + x4));
              v[x4] += b4.x; v[x4 + 1] += b4.y; v[x4 + 2] += b4.z; v[x4 + 3] += b4.w;
            }
          }
        }
        if (p.residual && grow < (long long)p.M) {
          const float *res = p.residual + (size_t)grow * p.N + col0;
#pragma unroll
          for (int x4 = 0; x4 < 32; x4 += 4) {
            if (col0 + x4 < (int)p.N) {
              const float4 r4 = __ldg(reinterpret_cast<const float4 *>(res + x4));
              v[x4] += r4.x; v[x4 + 1] += r4.y; v[x4 + 2] += r4.z; v[x4 + 3] += r4.w;
            }
          }
        }
        // the two staging slabs alternate over the stores actually issued; a slab is free once the store
        // issued two stores ago has read it
        auto emit = [&](const CUtensorMap *tm) -> bool {
          const uint32_t sb = n_store & 1;
          ++n_store;
          if (issuer) tma_store_wait_read_1();
          mbar_arrive(bar(EPI_A));
          if (!mbar_wait(bar(EPI_A), n_sync_a & 1, abort_flag)) return false;
          ++n_sync_a;
          uint8_t *stage = smem + kSmemStaging + sb * kSlabBytes + row * 128;
#pragma unroll
          for (int x = 0; x < 8; ++x)
            *reinterpret_cast<float4 *>(stage + ((x ^ (row & 7)) << 4)) = make_float4(v[4 * x], v[4 * x + 1], v[4 * x + 2], v[4 * x + 3]);
          fence_proxy_async_smem();
          mbar_arrive(bar(EPI_B));
          if (!mbar_wait(bar(EPI_B), n_sync_b & 1, abort_flag)) return false;
          ++n_sync_b;
          if (issuer) {
            tma_store_2d(tm, a0 + kSmemStaging + sb * kSlabBytes, col0, m_tile * TM);  // rows beyond M, columns beyond N are dropped
            tma_store_commit();
          }
          return true;
        };
        if (!p.gelu || p.store_pre) {
          if (!emit(to)) { ok = false; break; }
        }
        if (p.gelu) {
          // the activated output leaves through a second map; the pre-activation above is what the backward reads
#pragma unroll
          for (int x = 0; x < 32; ++x) v[x] = gelu_value(v[x]);
          if (!emit(&tmO1)) { ok = false; break; }
        }
      }
    }
    if (issuer) tma_store_wait_read_all();
  }

  // ---------------------------------------------------------------- teardown (all roles)
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (warp == 1) {
      commit_elected(bar(DRAIN));  // by the lane that issued the MMAs: the election is deterministic
      for (int n = 0; n < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++n) {
      }
    }
    if (warp == 0 && lane == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, DEV_STATUS_WAIT_EXPIRED);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

struct DeviceInfo {
  std::once_flag once;
  int n_sm = 0;
  bool ok = false;
};
DeviceInfo g_dev[64];

}  // namespace

bool tensor_linear_supported(const float *x, const float *const *w, const float *const *bias, float *const *out,
                             const float *residual, int n_mats, uint32_t M, uint32_t K, uint32_t N) {
  if (n_mats < 1 || n_mats > 3 || M == 0 || K == 0 || N == 0) return false;
  if ((K & 3u) || (N & 3u)) return false;  // row pitches must be multiples of 16 bytes
  uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual);
  for (int j = 0; j < n_mats; ++j)
    bits |= reinterpret_cast<uintptr_t>(w[j]) | reinterpret_cast<uintptr_t>(out[j]) | reinterpret_cast<uintptr_t>(bias ? bias[j] : nullptr);
  if (bits & 15u) return false;
  if ((uint64_t)M * K >= (1ull << 38) || (uint64_t)M * N >= (1ull << 38)) return false;
  return true;
}

int tensor_linear(const float *x, const float *const *w, const float *const *bias, float *const *out, const float *residual,
                  float *gelu_out, int n_mats, uint32_t M, uint32_t K, uint32_t N, cudaStream_t s) {
  if (gelu_out && (n_mats != 1 || residual || (reinterpret_cast<uintptr_t>(gelu_out) & 15u))) return DF_ERR_UNSUPPORTED;
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev)) != DF_OK || dev < 0 || dev >= 64) return DF_ERR_CUDA;
  DeviceInfo &di = g_dev[dev];
  std::call_once(di.once, [&]() {
    di.ok = cudaFuncSetAttribute(k_linear_tf32, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal) == cudaSuccess &&
            cudaDeviceGetAttribute(&di.n_sm, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && di.n_sm > 0;
  });
  if (!di.ok) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  CUtensorMap tmX, tmW[3], tmO[3];
  bool ok = encode_matrix_map(&tmX, x, M, K, TM, false);
  for (int j = 0; j < 3; ++j) {
    const int jj = j < n_mats ? j : 0;  // unused slots repeat the first matrix: every map is valid
    ok = ok && encode_matrix_map(&tmW[j], w[jj], N, K, TN, false) && encode_matrix_map(&tmO[j], out[jj], M, N, TM, true);
  }
  // with the GELU epilogue the second output map carries the activated values; a caller that does not want the
  // pre-activation passes out[0] == nullptr, and the first map then repeats the second (it is never stored through)
  if (gelu_out) ok = ok && encode_matrix_map(&tmO[1], gelu_out, M, N, TM, true);
  if (!ok) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  LinParams p;
  p.gelu = gelu_out ? 1 : 0;
  p.store_pre = (gelu_out && out[0] != gelu_out) ? 1 : 0;
  for (int j = 0; j < 3; ++j) p.bias[j] = (bias && j < n_mats) ? bias[j] : nullptr;
  p.residual = residual;
  p.M = M; p.N = N; p.K = K;
  p.n_mats = n_mats;
  p.n_tiles_per_mat = (int)((N + TN - 1) / TN);
  p.n_tiles_total = p.n_tiles_per_mat * n_mats;
  p.tiles = (long long)((M + TM - 1) / TM) * p.n_tiles_total;
  p.status = device_status_ptr();
  const dim3 grid((unsigned)(p.tiles < di.n_sm ? p.tiles : di.n_sm));
  k_linear_tf32<<<grid, kLinThreads, kSmemTotal, s>>>(tmX, tmW[0], tmW[1], tmW[2], tmO[0], tmO[1], tmO[2], p);
  note_launch();
  return check_cuda(cudaGetLastError());
}

}  // namespace df
