// attn_bwd_sm100.cu — fused causal attention backward for B200 (sm_100a), fp32 API, TF32 MMA.
//
// Replaces the arithmetic of kernel_mha_bwd_all_heads
// (darkforest-cuda/kernels/attention_fused.cu:390-516) from saved logsumexp and delta:
//   P = exp(scale*QK^T - lse)   dP = dO V^T   dS = P o (dP - delta)
//   dV = P^T dO                 dK = scale * dS^T Q        dQ = scale * dS K
// with no S x S scratch, no atomics (bit-reproducible) and no memsets: two kernels, first dK/dV,
// then dQ, each recomputing P tile by tile on the tensor cores.
//
// dK/dV kernel: a CTA owns 128 keys (TMEM lanes = keys) and walks the 128-query tiles that can see
//   them.  S^T = K Q^T and dP^T = V dO^T are SS MMAs (both operands K-major in shared memory);
//   eight compute warps (two per lane quarter, splitting the 128 query columns) turn S^T into P^T
//   and dP^T into dS^T in place in TMEM; dV += P^T dO and dK += dS^T Q are TS MMAs whose B operand
//   (dO, Q as [query, d]) is MN-major.  A 32-bit MN-major operand needs a different shared-memory
//   swizzle (32-byte atoms) than a K-major one, so Q and dO tiles are fetched twice by TMA, once
//   per layout, through four independently recycled buffers.
// dQ kernel: a CTA owns 128 queries (lanes = queries) and walks the key tiles they can see:
//   S = Q K^T, dP = dO V^T (SS), dS in TMEM, dQ += dS K (TS, K tile MN-major: K is fetched twice).
// The MMA issue order interleaves the two phases of consecutive tiles (.., dV_i, S_{i+1}, dK_i,
// dP_{i+1}, ..) so the tensor pipe has work while the compute warps are busy; single TMEM and
// shared-memory stages suffice because tcgen05 MMAs of one thread execute in issue order.
//
// Inputs are rounded to TF32 by the TFLOAT32 tensor maps (nearest even); P and dS are rounded
// with cvt.rna before they are written back to TMEM. Every wait is bounded (see mbar_wait).
#include <math.h>

#include "df_common.cuh"
#include "sm100_ptx.cuh"

namespace df {
namespace {

using namespace ptx;

constexpr int BT = 128;  // tile edge: keys per CTA / queries per step (and vice versa)
constexpr int HD = 64;
constexpr int kBwdThreads = 352;  // warps 0-7 compute, 8-9 TMA producers, 10 MMA issuer
constexpr uint32_t kSlab = 128 * 128;
constexpr uint32_t kTile = 2 * kSlab;
constexpr uint32_t kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  const float *lse;
  const float *delta;
  float *dq, *dk, *dv;
  uint32_t B, H, Sq, Sk;
  float scale, scale_log2;
  int causal;
  long long shift;
  unsigned int *status;
};

// 8 K-steps of a 128x128x64 SS MMA, both operands K-major tiles of two 128-byte slabs.
__device__ __forceinline__ void issue_ss_128x128(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem, uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < HD / 8; ++kk) {
    const uint32_t off = (kk >> 2) * kSlab + (kk & 3) * 32;
    mma_tf32_ss(d_tmem, make_smem_desc(a_smem + off, 16, 1024, kSwz128), make_smem_desc(b_smem + off, 16, 1024, kSwz128),
                idesc, kk > 0);
  }
}
// 16 K-steps of a 128x64x128 TS MMA: A = 128 TMEM columns, B = MN-major [128 rows (K), 64 dims (N)].
__device__ __forceinline__ void issue_ts_128x64(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_smem, uint32_t idesc,
                                                bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < BT / 8; ++kk)
    mma_tf32_ts(d_tmem, a_tmem + kk * 8, make_smem_desc(b_smem + kk * 1024, kSlab, 512, kSwz128B32), idesc,
                (accumulate || kk > 0) ? 1u : 0u);
}
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap *m, uint32_t bar, int h, int row0, int b) {
  mbar_arrive_expect_tx(bar, kTile);
  tma_load_4d(dst, m, bar, 0, h, row0, b);
  tma_load_4d(dst + kSlab, m, bar, 32, h, row0, b);
}

// =========================================================================================
// dK / dV
// =========================================================================================
namespace kv {
enum Bar { KV_FULL = 0, QK_FULL, QK_EMPTY, GK_FULL, GK_EMPTY, QM_FULL, QM_EMPTY, GM_FULL, GM_EMPTY,
           S_FULL, DP_FULL, P_FULL, DS_FULL, STAT_FULL, ACC_FULL, DRAIN, NUM };
constexpr uint32_t kStats = 6 * kTile;             // lse2[2][128], delta[2][128]
constexpr uint32_t kBars = kStats + 4 * 128 * 4;
constexpr uint32_t kSmemTotal = kBars + 256 + 1024;
}  // namespace kv

__global__ void __launch_bounds__(kBwdThreads, 1)
k_attn_bwd_dkdv_tf32_d64(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const __grid_constant__ CUtensorMap tmQk, const __grid_constant__ CUtensorMap tmGk,
                         const __grid_constant__ CUtensorMap tmQm, const __grid_constant__ CUtensorMap tmGm,
                         const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                         const BwdParams p) {
  using namespace kv;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aK = smem_u32(smem), aV = aK + kTile, aQk = aK + 2 * kTile, aGk = aK + 3 * kTile,
                 aQm = aK + 4 * kTile, aGm = aK + 5 * kTile;
  float *sLse2 = reinterpret_cast<float *>(smem + kStats);   // [2][128]
  float *sDelta = sLse2 + 256;                               // [2][128]
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kBars);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kBars + 128);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + kBars + 132);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid, (batch, head) fastest; key tile 0 sees the most queries, so all heads' tile 0 go first
  const uint32_t n_bh = p.B * p.H, bh = blockIdx.x % n_bh;
  const int kt = (int)(blockIdx.x / n_bh);
  const uint32_t b = bh / p.H, h = bh % p.H;
  const long long k0 = (long long)kt * BT;
  const size_t dm = (size_t)p.H * HD;

  long long q_first = p.causal ? k0 - p.shift : 0;
  if (q_first < 0) q_first = 0;
  const long long i_begin = q_first / BT;
  const long long n_qt = ((long long)p.Sq + BT - 1) / BT;
  const int n_it = (int)(n_qt - i_begin);

  if (n_it <= 0) {
    // no query sees these keys: dK = dV = 0
    if (warp < 8) {
      const long long kj = k0 + (warp & 3) * 32 + lane;
      if (kj < (long long)p.Sk) {
        float4 *dst = reinterpret_cast<float4 *>(((warp >> 2) ? p.dk : p.dv) + ((size_t)b * p.Sk + (size_t)kj) * dm + h * HD);
#pragma unroll
        for (int x = 0; x < HD / 4; ++x) dst[x] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    return;
  }

  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  if (warp == 8 && lane == 0) {
    // The first producer thread initialises the barriers itself and requests K, V and the first
    // query tile in all four layouts before the CTA-wide set-up barrier, so that the copies'
    // latency overlaps the tensor-memory allocation.
    for (int i = 0; i < NUM; ++i) mbar_init(bar(i), (i == P_FULL || i == DS_FULL || i == STAT_FULL) ? 256 : 1);
    *abort_flag = 0;
    mbar_init_fence();
    mbar_arrive_expect_tx(bar(KV_FULL), 2 * kTile);
    tma_load_4d(aK, &tmK, bar(KV_FULL), 0, (int)h, (int)k0, (int)b);
    tma_load_4d(aK + kSlab, &tmK, bar(KV_FULL), 32, (int)h, (int)k0, (int)b);
    tma_load_4d(aV, &tmV, bar(KV_FULL), 0, (int)h, (int)k0, (int)b);
    tma_load_4d(aV + kSlab, &tmV, bar(KV_FULL), 32, (int)h, (int)k0, (int)b);
    const int q0 = (int)(i_begin * BT);
    load_tile(aQk, &tmQk, bar(QK_FULL), (int)h, q0, (int)b);
    load_tile(aGk, &tmGk, bar(GK_FULL), (int)h, q0, (int)b);
    load_tile(aGm, &tmGm, bar(GM_FULL), (int)h, q0, (int)b);
    load_tile(aQm, &tmQm, bar(QM_FULL), (int)h, q0, (int)b);
  }
  if (warp == 10) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const uint32_t tS = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 320;

  if (warp == 8) {
    // ---------------------------------------------- producer: K-major Q and dO tiles (tile 0 is on its way)
    if (lane == 0) {
      for (int it = 1; it < n_it; ++it) {
        const int q0 = (int)((i_begin + it) * BT);
        if (!mbar_wait(bar(QK_EMPTY), (it - 1) & 1, abort_flag)) break;
        load_tile(aQk, &tmQk, bar(QK_FULL), (int)h, q0, (int)b);
        if (!mbar_wait(bar(GK_EMPTY), (it - 1) & 1, abort_flag)) break;
        load_tile(aGk, &tmGk, bar(GK_FULL), (int)h, q0, (int)b);
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------- producer: MN-major dO and Q tiles
    if (lane == 0) {
      for (int it = 1; it < n_it; ++it) {
        const int q0 = (int)((i_begin + it) * BT);
        if (!mbar_wait(bar(GM_EMPTY), (it - 1) & 1, abort_flag)) break;
        load_tile(aGm, &tmGm, bar(GM_FULL), (int)h, q0, (int)b);
        if (!mbar_wait(bar(QM_EMPTY), (it - 1) & 1, abort_flag)) break;
        load_tile(aQm, &tmQm, bar(QM_FULL), (int)h, q0, (int)b);
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_ss = make_idesc(kFmtTF32, BT, BT, 0, 0);
      const uint32_t idesc_ts = make_idesc(kFmtTF32, BT, HD, 0, 1);
      bool ok = mbar_wait(bar(KV_FULL), 0, abort_flag);
      ok = ok && mbar_wait(bar(QK_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_ss_128x128(tS, aK, aQk, idesc_ss);  // S^T_0 = K Q^T
        mma_commit(bar(S_FULL));
        mma_commit(bar(QK_EMPTY));
        ok = mbar_wait(bar(GK_FULL), 0, abort_flag);
      }
      if (ok) {
        tc_fence_after_sync();
        issue_ss_128x128(tDP, aV, aGk, idesc_ss);  // dP^T_0 = V dO^T
        mma_commit(bar(DP_FULL));
        mma_commit(bar(GK_EMPTY));
      }
      for (int it = 0; ok && it < n_it; ++it) {
        const uint32_t ph = it & 1, nph = (it + 1) & 1;
        if (!mbar_wait(bar(P_FULL), ph, abort_flag) || !mbar_wait(bar(GM_FULL), ph, abort_flag)) break;
        tc_fence_after_sync();
        issue_ts_128x64(tDV, tS, aGm, idesc_ts, it > 0);  // dV += P^T dO
        mma_commit(bar(GM_EMPTY));
        if (it + 1 < n_it) {
          if (!mbar_wait(bar(QK_FULL), nph, abort_flag)) break;
          tc_fence_after_sync();
          issue_ss_128x128(tS, aK, aQk, idesc_ss);  // S^T_{i+1} (overwrites P^T_i after dV_i has read it)
          mma_commit(bar(S_FULL));
          mma_commit(bar(QK_EMPTY));
        }
        if (!mbar_wait(bar(DS_FULL), ph, abort_flag) || !mbar_wait(bar(QM_FULL), ph, abort_flag)) break;
        tc_fence_after_sync();
        issue_ts_128x64(tDK, tDP, aQm, idesc_ts, it > 0);  // dK += dS^T Q
        mma_commit(bar(QM_EMPTY));
        if (it + 1 < n_it) {
          if (!mbar_wait(bar(GK_FULL), nph, abort_flag)) break;
          tc_fence_after_sync();
          issue_ss_128x128(tDP, aV, aGk, idesc_ss);  // dP^T_{i+1}
          mma_commit(bar(DP_FULL));
          mma_commit(bar(GK_EMPTY));
        }
      }
      mma_commit(bar(ACC_FULL));
    }
  } else {
    // ---------------------------------------------- compute warps: lanes = keys, columns = queries
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const int tid = threadIdx.x;  // 0..255
    const long long kj = k0 + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int col0 = half * 64;
    const size_t s_base = ((size_t)b * p.H + h) * p.Sq;
    // row statistics of the query tile: threads 0-127 fetch lse, 128-255 fetch delta
    auto fetch_stat = [&](int it) -> float {
      const long long q = (i_begin + it) * BT + (tid & 127);
      if (it >= n_it || q >= (long long)p.Sq) return (tid < 128) ? INFINITY : 0.0f;
      if (tid < 128) {
        const float v = __ldg(p.lse + s_base + q);
        return (v == -INFINITY) ? INFINITY : v * kLog2e;  // rows without visible keys give P = 0
      }
      return __ldg(p.delta + s_base + q);
    };
    float stat_next = fetch_stat(0);
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const uint32_t ph = it & 1;
      const long long q0 = (i_begin + it) * BT;
      float *lse2 = sLse2 + ph * 128, *dlt = sDelta + ph * 128;
      if (tid < 128) lse2[tid] = stat_next; else dlt[tid - 128] = stat_next;
      // publish the staged statistics to the other compute threads (bounded, like every wait here)
      mbar_arrive(bar(STAT_FULL));
      if (!mbar_wait(bar(STAT_FULL), ph, abort_flag)) { ok = false; break; }
      stat_next = fetch_stat(it + 1);
      // visible iff key <= query + shift  <=>  column >= kj - shift - q0
      const bool need_mask = p.causal && (q0 + p.shift < k0 + (BT - 1));
      long long cmin_ll = kj - p.shift - q0;
      const int cmin = !need_mask ? 0 : (cmin_ll > BT ? BT : (cmin_ll < 0 ? 0 : (int)cmin_ll));
      if (!mbar_wait(bar(S_FULL), ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      float pr[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + lane_base + col0 + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int col = col0 + c * 32 + x;
          float e = ex2_approx(fmaf(__uint_as_float(r[x]), p.scale_log2, -lse2[col]));
          if (col < cmin) e = 0.0f;
          r[x] = cvt_rna_tf32(e);
          pr[c * 32 + x] = __uint_as_float(r[x]);
        }
        tmem_st32(tS + lane_base + col0 + c * 32, r);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(P_FULL));
      if (!mbar_wait(bar(DP_FULL), ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tDP + lane_base + col0 + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int col = col0 + c * 32 + x;
          r[x] = cvt_rna_tf32(pr[c * 32 + x] * (__uint_as_float(r[x]) - dlt[col]));
        }
        tmem_st32(tDP + lane_base + col0 + c * 32, r);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(DS_FULL));
    }
    if (ok && mbar_wait(bar(ACC_FULL), 0, abort_flag)) {
      tc_fence_after_sync();
      // Warps 0-3 hand over dV, warps 4-7 scale * dK. Every MMA has finished, so the K tile's
      // shared memory stages dV and the V tile's dK, in the 128-byte-swizzled slab layout of the
      // store's tensor map (16-byte chunk c of row r at c ^ (r % 8)); the copy engine then
      // writes the two tiles and drops key rows beyond Sk.
      const float mul = half ? p.scale : 1.0f;
      uint8_t *stage = smem + half * kTile + row * 128;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32((half ? tDK : tDV) + lane_base + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 8; ++x)
          *reinterpret_cast<float4 *>(stage + c * kSlab + ((x ^ (row & 7)) << 4)) =
              make_float4(__uint_as_float(r[4 * x]) * mul, __uint_as_float(r[4 * x + 1]) * mul,
                          __uint_as_float(r[4 * x + 2]) * mul, __uint_as_float(r[4 * x + 3]) * mul);
      }
      fence_proxy_async_smem();
      mbar_arrive(bar(STAT_FULL));  // phase n_it of the statistics barrier: all 256 threads have staged
      if (tid == 0 && mbar_wait(bar(STAT_FULL), n_it & 1, abort_flag)) {
        tma_store_4d(&tmDV, aK, 0, (int)h, (int)k0, (int)b);
        tma_store_4d(&tmDV, aK + kSlab, 32, (int)h, (int)k0, (int)b);
        tma_store_4d(&tmDK, aV, 0, (int)h, (int)k0, (int)b);
        tma_store_4d(&tmDK, aV + kSlab, 32, (int)h, (int)k0, (int)b);
        tma_store_commit();
        tma_store_wait_read_all();
      }
    }
  }

  // ---------------------------------------------------------------- teardown (all roles)
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (warp == 10 && lane == 0) {
      mma_commit(bar(DRAIN));
      for (int t = 0; t < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++t) {
      }
    }
    if ((warp == 8 || warp == 9) && lane == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, DEV_STATUS_WAIT_EXPIRED);
    __syncthreads();
  }
  if (warp == 10) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// =========================================================================================
// dQ
// =========================================================================================
namespace dq {
enum Bar { QG_FULL = 0, KK_FULL, KK_EMPTY, VK_FULL, VK_EMPTY, KM_FULL, KM_EMPTY, S_FULL, S_FREE, DP_FULL, DS_FULL,
           ACC_FULL, DRAIN, NUM };
constexpr uint32_t kBars = 5 * kTile;
constexpr uint32_t kSmemTotal = kBars + 256 + 1024;
}  // namespace dq

__global__ void __launch_bounds__(kBwdThreads, 1)
k_attn_bwd_dq_tf32_d64(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
                       const __grid_constant__ CUtensorMap tmKk, const __grid_constant__ CUtensorMap tmVk,
                       const __grid_constant__ CUtensorMap tmKm, const __grid_constant__ CUtensorMap tmDQ,
                       const BwdParams p) {
  using namespace dq;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aQ = smem_u32(smem), aG = aQ + kTile, aKk = aQ + 2 * kTile, aVk = aQ + 3 * kTile, aKm = aQ + 4 * kTile;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kBars);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kBars + 128);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + kBars + 132);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid, (batch, head) fastest; heaviest (latest) query tile of every head first
  const uint32_t n_bh = p.B * p.H, bh = blockIdx.x % n_bh;
  const int qt = (int)(gridDim.x / n_bh) - 1 - (int)(blockIdx.x / n_bh);
  const uint32_t b = bh / p.H, h = bh % p.H;
  const long long q0 = (long long)qt * BT;
  const size_t dm = (size_t)p.H * HD;

  long long kv_end = p.causal ? q0 + (BT - 1) + p.shift + 1 : (long long)p.Sk;
  if (kv_end > (long long)p.Sk) kv_end = p.Sk;
  if (kv_end < 0) kv_end = 0;
  const int n_kv = (int)((kv_end + BT - 1) / BT);

  if (n_kv == 0) {
    if (warp < 8) {
      const long long i = q0 + (warp & 3) * 32 + lane;
      if (i < (long long)p.Sq) {
        float4 *dst = reinterpret_cast<float4 *>(p.dq + ((size_t)b * p.Sq + (size_t)i) * dm + h * HD + (warp >> 2) * 32);
#pragma unroll
        for (int x = 0; x < 8; ++x) dst[x] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    return;
  }

  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  if (warp == 8 && lane == 0) {
    // barriers and the first copies (Q, dO, key tile 0 in its three roles) before the set-up barrier
    for (int i = 0; i < NUM; ++i) mbar_init(bar(i), (i == S_FREE || i == DS_FULL) ? 256 : 1);
    *abort_flag = 0;
    mbar_init_fence();
    mbar_arrive_expect_tx(bar(QG_FULL), 2 * kTile);
    tma_load_4d(aQ, &tmQ, bar(QG_FULL), 0, (int)h, (int)q0, (int)b);
    tma_load_4d(aQ + kSlab, &tmQ, bar(QG_FULL), 32, (int)h, (int)q0, (int)b);
    tma_load_4d(aG, &tmG, bar(QG_FULL), 0, (int)h, (int)q0, (int)b);
    tma_load_4d(aG + kSlab, &tmG, bar(QG_FULL), 32, (int)h, (int)q0, (int)b);
    load_tile(aKk, &tmKk, bar(KK_FULL), (int)h, 0, (int)b);
    load_tile(aVk, &tmVk, bar(VK_FULL), (int)h, 0, (int)b);
    load_tile(aKm, &tmKm, bar(KM_FULL), (int)h, 0, (int)b);
  }
  if (warp == 10) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const uint32_t tS = tmem, tDP = tmem + 128, tDQ = tmem + 256;

  if (warp == 8) {
    if (lane == 0) {
      for (int j = 1; j < n_kv; ++j) {
        if (!mbar_wait(bar(KK_EMPTY), (j - 1) & 1, abort_flag)) break;
        load_tile(aKk, &tmKk, bar(KK_FULL), (int)h, j * BT, (int)b);
        if (!mbar_wait(bar(VK_EMPTY), (j - 1) & 1, abort_flag)) break;
        load_tile(aVk, &tmVk, bar(VK_FULL), (int)h, j * BT, (int)b);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      for (int j = 1; j < n_kv; ++j) {
        if (!mbar_wait(bar(KM_EMPTY), (j - 1) & 1, abort_flag)) break;
        load_tile(aKm, &tmKm, bar(KM_FULL), (int)h, j * BT, (int)b);
      }
    }
  } else if (warp == 10) {
    if (lane == 0) {
      const uint32_t idesc_ss = make_idesc(kFmtTF32, BT, BT, 0, 0);
      const uint32_t idesc_ts = make_idesc(kFmtTF32, BT, HD, 0, 1);
      bool ok = mbar_wait(bar(QG_FULL), 0, abort_flag);
      ok = ok && mbar_wait(bar(KK_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_ss_128x128(tS, aQ, aKk, idesc_ss);  // S_0 = Q K^T
        mma_commit(bar(S_FULL));
        mma_commit(bar(KK_EMPTY));
        ok = mbar_wait(bar(VK_FULL), 0, abort_flag);
      }
      if (ok) {
        tc_fence_after_sync();
        issue_ss_128x128(tDP, aG, aVk, idesc_ss);  // dP_0 = dO V^T
        mma_commit(bar(DP_FULL));
        mma_commit(bar(VK_EMPTY));
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const uint32_t ph = j & 1, nph = (j + 1) & 1;
        if (j + 1 < n_kv) {
          if (!mbar_wait(bar(S_FREE), ph, abort_flag) || !mbar_wait(bar(KK_FULL), nph, abort_flag)) break;
          tc_fence_after_sync();
          issue_ss_128x128(tS, aQ, aKk, idesc_ss);  // S_{j+1}: P_j already lives in registers
          mma_commit(bar(S_FULL));
          mma_commit(bar(KK_EMPTY));
        }
        if (!mbar_wait(bar(DS_FULL), ph, abort_flag) || !mbar_wait(bar(KM_FULL), ph, abort_flag)) break;
        tc_fence_after_sync();
        issue_ts_128x64(tDQ, tDP, aKm, idesc_ts, j > 0);  // dQ += dS K
        mma_commit(bar(KM_EMPTY));
        if (j + 1 < n_kv) {
          if (!mbar_wait(bar(VK_FULL), nph, abort_flag)) break;
          tc_fence_after_sync();
          issue_ss_128x128(tDP, aG, aVk, idesc_ss);  // dP_{j+1} (overwrites dS_j after dQ_j has read it)
          mma_commit(bar(DP_FULL));
          mma_commit(bar(VK_EMPTY));
        }
      }
      mma_commit(bar(ACC_FULL));
    }
  } else {
    // ---------------------------------------------- compute warps: lanes = queries, columns = keys
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const long long i = q0 + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int col0 = half * 64;
    const bool row_ok = i < (long long)p.Sq;
    const size_t s_idx = ((size_t)b * p.H + h) * p.Sq + (size_t)(row_ok ? i : 0);
    float lse2 = INFINITY, dlt = 0.0f;
    if (row_ok) {
      const float v = __ldg(p.lse + s_idx);
      lse2 = (v == -INFINITY) ? INFINITY : v * kLog2e;
      dlt = __ldg(p.delta + s_idx);
    }
    long long kmax_ll = p.causal ? i + p.shift + 1 : (long long)p.Sk;
    if (kmax_ll > (long long)p.Sk) kmax_ll = p.Sk;
    if (kmax_ll < 0) kmax_ll = 0;
    const int kmax = (int)kmax_ll;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const uint32_t ph = j & 1;
      const int key0 = j * BT;
      const bool need_mask = key0 + BT > kmax;
      if (!mbar_wait(bar(S_FULL), ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      float pr[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + lane_base + col0 + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          float e = ex2_approx(fmaf(__uint_as_float(r[x]), p.scale_log2, -lse2));
          if (need_mask && !(key0 + col0 + c * 32 + x < kmax)) e = 0.0f;
          pr[c * 32 + x] = e;
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bar(S_FREE));
      if (!mbar_wait(bar(DP_FULL), ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tDP + lane_base + col0 + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 32; ++x) r[x] = cvt_rna_tf32(pr[c * 32 + x] * (__uint_as_float(r[x]) - dlt));
        tmem_st32(tDP + lane_base + col0 + c * 32, r);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(DS_FULL));
    }
    if (ok && mbar_wait(bar(ACC_FULL), 0, abort_flag)) {
      tc_fence_after_sync();
      uint32_t r[32];
      tmem_ld32(tDQ + lane_base + half * 32, r);  // each half handles 32 of the 64 dims = one 128-byte slab
      tmem_wait_ld();
      // staged over the Q tile (free: every MMA has finished) in the swizzled slab layout of the
      // store's tensor map, then written by the copy engine, which drops rows beyond Sq
      uint8_t *stage = smem + half * kSlab + row * 128;
#pragma unroll
      for (int x = 0; x < 8; ++x)
        *reinterpret_cast<float4 *>(stage + ((x ^ (row & 7)) << 4)) =
            make_float4(__uint_as_float(r[4 * x]) * p.scale, __uint_as_float(r[4 * x + 1]) * p.scale,
                        __uint_as_float(r[4 * x + 2]) * p.scale, __uint_as_float(r[4 * x + 3]) * p.scale);
      fence_proxy_async_smem();
      mbar_arrive(bar(DS_FULL));  // phase n_kv of the dS barrier: all 256 threads have staged
      if (threadIdx.x == 0 && mbar_wait(bar(DS_FULL), n_kv & 1, abort_flag)) {
        tma_store_4d(&tmDQ, aQ, 0, (int)h, (int)q0, (int)b);
        tma_store_4d(&tmDQ, aQ + kSlab, 32, (int)h, (int)q0, (int)b);
        tma_store_commit();
        tma_store_wait_read_all();
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (warp == 10 && lane == 0) {
      mma_commit(bar(DRAIN));
      for (int t = 0; t < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++t) {
      }
    }
    if ((warp == 8 || warp == 9) && lane == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, DEV_STATUS_WAIT_EXPIRED);
    __syncthreads();
  }
  if (warp == 10) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

bool tensor_backward_supported(const AttnParams &p) {
  if (env_flag("DF_ATTN_DISABLE_TENSOR", 0) || env_flag("DF_ATTN_DISABLE_TENSOR_BWD", 0)) return false;
  if (p.D != HD || p.Sk == 0 || p.Sq == 0 || p.B == 0) return false;
  if (!(p.scale > 0.0f) || !isfinite(p.scale)) return false;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                         reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.d_out) |
                         reinterpret_cast<uintptr_t>(p.d_q) | reinterpret_cast<uintptr_t>(p.d_k) |
                         reinterpret_cast<uintptr_t>(p.d_v);
  if (bits & 15u) return false;
  if ((uint64_t)p.B * p.H * ((uint64_t)(p.Sq > p.Sk ? p.Sq : p.Sk) / BT + 1) > 0x7fffffffull) return false;
  if ((uint64_t)p.Sq * p.H * HD * 4 >= (1ull << 40) || (uint64_t)p.Sk * p.H * HD * 4 >= (1ull << 40)) return false;
  if (p.shift > (1ll << 40) || p.shift < -(1ll << 40)) return false;
  return true;
}

int tensor_backward(const AttnParams &p, cudaStream_t s) {
  static bool attr_set[64] = {false};
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev)) != DF_OK) return DF_ERR_CUDA;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(k_attn_bwd_dkdv_tf32_d64, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kv::kSmemTotal)) != DF_OK ||
        check_cuda(cudaFuncSetAttribute(k_attn_bwd_dq_tf32_d64, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)dq::kSmemTotal)) != DF_OK)
      return DF_ERR_CUDA;
    attr_set[dev] = true;
  }
  CUtensorMap tmQk, tmQm, tmGk, tmGm, tmKk, tmKm, tmVk, tmDQ, tmDK, tmDV;
  if (!encode_head_tile_map(&tmQk, p.q, false, HD, p.B, p.H, p.Sq, BT, false) ||
      !encode_head_tile_map(&tmQm, p.q, false, HD, p.B, p.H, p.Sq, BT, true) ||
      !encode_head_tile_map(&tmGk, p.d_out, false, HD, p.B, p.H, p.Sq, BT, false) ||
      !encode_head_tile_map(&tmGm, p.d_out, false, HD, p.B, p.H, p.Sq, BT, true) ||
      !encode_head_tile_map(&tmKk, p.k, false, HD, p.B, p.H, p.Sk, BT, false) ||
      !encode_head_tile_map(&tmKm, p.k, false, HD, p.B, p.H, p.Sk, BT, true) ||
      !encode_head_tile_map(&tmVk, p.v, false, HD, p.B, p.H, p.Sk, BT, false) ||
      !encode_head_tile_map(&tmDQ, p.d_q, false, HD, p.B, p.H, p.Sq, BT, false, true) ||
      !encode_head_tile_map(&tmDK, p.d_k, false, HD, p.B, p.H, p.Sk, BT, false, true) ||
      !encode_head_tile_map(&tmDV, p.d_v, false, HD, p.B, p.H, p.Sk, BT, false, true)) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  BwdParams bp;
  bp.lse = p.lse_in;
  bp.delta = p.delta_in;
  bp.dq = p.d_q; bp.dk = p.d_k; bp.dv = p.d_v;
  bp.B = p.B; bp.H = p.H; bp.Sq = p.Sq; bp.Sk = p.Sk;
  bp.scale = p.scale;
  bp.scale_log2 = p.scale * kLog2e;
  bp.causal = p.causal;
  bp.shift = p.shift;
  bp.status = device_status_ptr();
  // measurement aid: DF_ATTN_BWD_PART=1 launches only the dK/dV kernel, =2 only the dQ kernel, so that a
  // benchmark can time each with events (the untouched gradients are then left as they were)
  const int part = env_flag("DF_ATTN_BWD_PART", 0);
  const dim3 grid_kv(((p.Sk + BT - 1) / BT) * p.B * p.H);
  const dim3 grid_q(((p.Sq + BT - 1) / BT) * p.B * p.H);
  // The two kernels are independent of each other. With one CTA per SM each, running them on two
  // streams lets the tail of one fill with CTAs of the other. The side stream and its two events
  // are created once per device (first call) and reused: fork after everything already queued on
  // `s`, join back into `s`, so callers see ordinary stream semantics (and it stays capturable).
  struct Side { cudaStream_t stream = nullptr; cudaEvent_t fork = nullptr, join = nullptr; bool ok = false; };
  static Side side[64];
  Side *sd = (dev >= 0 && dev < 64) ? &side[dev] : nullptr;
  if (sd && !sd->ok && env_flag("DF_ATTN_BWD_OVERLAP", 1)) {
    if (cudaStreamCreateWithFlags(&sd->stream, cudaStreamNonBlocking) == cudaSuccess &&
        cudaEventCreateWithFlags(&sd->fork, cudaEventDisableTiming) == cudaSuccess &&
        cudaEventCreateWithFlags(&sd->join, cudaEventDisableTiming) == cudaSuccess)
      sd->ok = true;
  }
  const bool overlap = part == 0 && sd && sd->ok && env_flag("DF_ATTN_BWD_OVERLAP", 1);
  cudaStream_t s_dq = s;
  if (overlap) {
    if (check_cuda(cudaEventRecord(sd->fork, s)) != DF_OK || check_cuda(cudaStreamWaitEvent(sd->stream, sd->fork, 0)) != DF_OK)
      return DF_ERR_CUDA;
    s_dq = sd->stream;
  }
  if (part != 2) {
    k_attn_bwd_dkdv_tf32_d64<<<grid_kv, kBwdThreads, kv::kSmemTotal, s>>>(tmKk, tmVk, tmQk, tmGk, tmQm, tmGm, tmDK, tmDV, bp);
    note_launch();
    if (check_cuda(cudaGetLastError()) != DF_OK) return DF_ERR_CUDA;
  }
  if (part != 1) {
    k_attn_bwd_dq_tf32_d64<<<grid_q, kBwdThreads, dq::kSmemTotal, s_dq>>>(tmQk, tmGk, tmKk, tmVk, tmKm, tmDQ, bp);
    note_launch();
    if (check_cuda(cudaGetLastError()) != DF_OK) return DF_ERR_CUDA;
  }
  if (overlap) {
    if (check_cuda(cudaEventRecord(sd->join, sd->stream)) != DF_OK || check_cuda(cudaStreamWaitEvent(s, sd->join, 0)) != DF_OK)
      return DF_ERR_CUDA;
  }
  return DF_OK;
}

}  // namespace df
