// attn_bwd_bf16_sm100.cu — bf16 variant of the attention backward for B200 (sm_100a).
//
// Same mathematics and the same two-kernel split (dK/dV, then dQ) as attn_bwd_sm100.cu, which
// replaces kernel_mha_bwd_all_heads (darkforest-cuda/kernels/attention_fused.cu:390-516); the
// reference has no bf16 attention. Differences that come with 16-bit operands:
//   * MMAs are kind::f16 with bf16 inputs and fp32 accumulation, 16 K-elements per instruction;
//   * a 16-bit MN-major operand uses the same 128-byte swizzle as a K-major one, so every Q, dO, K
//     tile is fetched ONCE and serves both roles; the freed shared memory holds two-stage rings;
//   * P^T and dS^T go back to TMEM as packed bf16 pairs: 128 rows of the other sequence take 64
//     columns, and each compute thread packs into the first half of the columns it has itself read
//     (columns [0,32) and [64,96)), so nobody overwrites scores another thread still needs;
//   * head dimension 64 or 128 (template parameter); gradients are written as bf16.
// Every wait is bounded (mbar_wait); there is no TMA multicast.
#include <math.h>

#include "df_common.cuh"
#include "sm100_ptx.cuh"

namespace df {
namespace {

using namespace ptx;

constexpr int BT = 128;
constexpr int kThreads = 352;  // warps 0-7 compute, 8-9 TMA producers, 10 MMA issuer
constexpr uint32_t kSlab = 128 * 128;
constexpr uint32_t kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;

struct Bwd16Params {
  const float *lse;
  const float *delta;
  void *dq, *dk, *dv;   // bf16 or fp32 elements, see Cfg16::OUT_F32
  uint32_t B, H, Sq, Sk;
  float scale, scale_log2;
  int causal;
  long long shift;
  unsigned int *status;
};

template <int HD_, bool OUT_F32_ = false>
struct Cfg16 {
  static constexpr int HD = HD_;
  static constexpr bool OUT_F32 = OUT_F32_;                // gradients as fp32 (ring partials) instead of bf16
  static constexpr uint32_t kOutElt = OUT_F32_ ? 4 : 2;
  static constexpr uint32_t kSlabs = HD_ * 2 / 128;        // 1 (D=64) or 2 (D=128)
  static constexpr uint32_t kTile = kSlabs * kSlab;        // 128 rows x HD bf16
  static constexpr int kKSteps = HD_ / 16;                 // K-steps of an SS MMA over the head dimension
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// The issue helpers are called by ALL lanes of the MMA warp; one elected lane issues each instruction (see elect_one).
// [128 x 128] = A[128 x HD] * B[128 x HD]^T, both K-major tiles of kSlabs 128-byte slabs.
template <class C>
__device__ __forceinline__ void issue_ss(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < C::kKSteps; ++kk) {
    const uint64_t off = (uint64_t)(((kk >> 2) * kSlab + (kk & 3) * 32) >> 4);
    if (elect_one()) mma_f16_ss(d_tmem, da + off, db + off, idesc, kk > 0);
  }
}
// [128 x HD] (+)= A[128 x 128 packed bf16 in TMEM] * B[128 rows (K) x HD (N), MN-major].
// The packed A operand lives in columns [0,32) and [64,96) of its 128-column region.
template <class C>
__device__ __forceinline__ void issue_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    if (elect_one())
      mma_f16_ts(d_tmem, a_tmem + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8), db + (uint64_t)(kk * (2048 >> 4)), idesc,
                 (accumulate || kk > 0) ? 1u : 0u);
}
template <class C>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap *m, uint32_t bar, int h, int row0, int b) {
  mbar_arrive_expect_tx(bar, C::kTile);
  for (uint32_t sl = 0; sl < C::kSlabs; ++sl) tma_load_4d(dst + sl * kSlab, m, bar, (int)(sl * 64), h, row0, b);
}
// 32 fp32 accumulator columns -> 32 fp32 values (128 bytes) in global memory
__device__ __forceinline__ void store_f32x32(uint8_t *dst, const uint32_t (&r)[32], float mul) {
  float4 *d4 = reinterpret_cast<float4 *>(dst);
#pragma unroll
  for (int x = 0; x < 8; ++x)
    d4[x] = make_float4(__uint_as_float(r[4 * x]) * mul, __uint_as_float(r[4 * x + 1]) * mul,
                        __uint_as_float(r[4 * x + 2]) * mul, __uint_as_float(r[4 * x + 3]) * mul);
}
// 32 fp32 accumulator columns -> 32 bf16 values (64 bytes) in global memory
__device__ __forceinline__ void store_bf16x32(uint8_t *dst, const uint32_t (&r)[32], float mul) {
  uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll
  for (int x = 0; x < 4; ++x)
    d4[x] = make_uint4(pack2(__uint_as_float(r[8 * x]) * mul, __uint_as_float(r[8 * x + 1]) * mul),
                       pack2(__uint_as_float(r[8 * x + 2]) * mul, __uint_as_float(r[8 * x + 3]) * mul),
                       pack2(__uint_as_float(r[8 * x + 4]) * mul, __uint_as_float(r[8 * x + 5]) * mul),
                       pack2(__uint_as_float(r[8 * x + 6]) * mul, __uint_as_float(r[8 * x + 7]) * mul));
}

// =========================================================================================
// dK / dV  (a CTA owns 128 keys; TMEM lanes = keys, columns = queries)
// =========================================================================================
namespace kv16 {
enum Bar { KV_FULL = 0, Q_FULL = 1, Q_EMPTY = 3, G_FULL = 5, G_EMPTY = 7,   // + ring stage
           S_FULL = 9, DP_FULL, P_FULL, DS_FULL, STAT_FULL, ACC_FULL, DRAIN, NUM };
template <class C> __host__ __device__ constexpr uint32_t stats_off() { return 6 * C::kTile; }   // K, V, Q[2], dO[2]
template <class C> __host__ __device__ constexpr uint32_t bars_off() { return stats_off<C>() + 4 * 128 * 4; }
template <class C> __host__ __device__ constexpr uint32_t smem_total() { return bars_off<C>() + 256 + 1024; }
}  // namespace kv16

template <class C>
__global__ void __launch_bounds__(kThreads, 1)
k_attn_bwd_dkdv_bf16(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG, const Bwd16Params p) {
  using namespace kv16;
  constexpr int HD = C::HD;
  constexpr uint32_t kTile = C::kTile;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aK = smem_u32(smem), aV = aK + kTile, aQ = aK + 2 * kTile, aG = aK + 4 * kTile;  // rings: + stage * kTile
  float *sLse2 = reinterpret_cast<float *>(smem + stats_off<C>());
  float *sDelta = sLse2 + 256;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + bars_off<C>());
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + bars_off<C>() + 160);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + bars_off<C>() + 164);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n_bh = p.B * p.H, bh = blockIdx.x % n_bh;
  const int kt = (int)(blockIdx.x / n_bh);  // key tile 0 sees the most queries: all heads' tile 0 go first
  const uint32_t b = bh / p.H, h = bh % p.H;
  const long long k0 = (long long)kt * BT;
  const size_t dm = (size_t)p.H * HD;

  long long q_first = p.causal ? k0 - p.shift : 0;
  if (q_first < 0) q_first = 0;
  const long long i_begin = q_first / BT;
  const int n_it = (int)(((long long)p.Sq + BT - 1) / BT - i_begin);

  if (n_it <= 0) {  // no query sees these keys: dK = dV = 0
    if (warp < 8) {
      const long long kj = k0 + (warp & 3) * 32 + lane;
      if (kj < (long long)p.Sk) {
        uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>((warp >> 2) ? p.dk : p.dv) +
                                               (((size_t)b * p.Sk + (size_t)kj) * dm + h * HD) * C::kOutElt);
#pragma unroll
        for (int x = 0; x < (int)(HD * C::kOutElt / 16); ++x) dst[x] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    return;
  }

  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM; ++i) mbar_init(bar(i), (i == P_FULL || i == DS_FULL || i == STAT_FULL) ? 256 : 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 10) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const uint32_t tS = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 256 + HD;

  if (warp == 8) {
    // producer: K, V once, then the Q ring
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(KV_FULL), 2 * kTile);
      for (uint32_t sl = 0; sl < C::kSlabs; ++sl) {
        tma_load_4d(aK + sl * kSlab, &tmK, bar(KV_FULL), (int)(sl * 64), (int)h, (int)k0, (int)b);
        tma_load_4d(aV + sl * kSlab, &tmV, bar(KV_FULL), (int)(sl * 64), (int)h, (int)k0, (int)b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1, use = it >> 1;
        if (use > 0 && !mbar_wait(bar(Q_EMPTY + s), (use - 1) & 1, abort_flag)) break;
        load_tile<C>(aQ + s * kTile, &tmQ, bar(Q_FULL + s), (int)h, (int)((i_begin + it) * BT), (int)b);
      }
    }
  } else if (warp == 9) {
    // producer: the dO ring
    if (lane == 0) {
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1, use = it >> 1;
        if (use > 0 && !mbar_wait(bar(G_EMPTY + s), (use - 1) & 1, abort_flag)) break;
        load_tile<C>(aG + s * kTile, &tmG, bar(G_FULL + s), (int)h, (int)((i_begin + it) * BT), (int)b);
      }
    }
  } else if (warp == 10) {
    // The whole warp runs this role, warp-uniformly; one elected lane issues the MMA and commit instructions and
    // every wait returns the same answer in all lanes (see elect_one).
    {
      const uint32_t idesc_ss = make_idesc(kFmtBF16, BT, BT, 0, 0);
      const uint32_t idesc_ts = make_idesc(kFmtBF16, BT, HD, 0, 1);
      const uint64_t dK = make_smem_desc(aK, 16, 1024, kSwz128), dV = make_smem_desc(aV, 16, 1024, kSwz128);
      // the same Q / dO tile serves as K-major B (S^T, dP^T) and as MN-major B (dK, dV)
      const uint64_t dQk[2] = {make_smem_desc(aQ, 16, 1024, kSwz128), make_smem_desc(aQ + kTile, 16, 1024, kSwz128)};
      const uint64_t dGk[2] = {make_smem_desc(aG, 16, 1024, kSwz128), make_smem_desc(aG + kTile, 16, 1024, kSwz128)};
      const uint64_t dQm[2] = {make_smem_desc(aQ, kSlab, 1024, kSwz128), make_smem_desc(aQ + kTile, kSlab, 1024, kSwz128)};
      const uint64_t dGm[2] = {make_smem_desc(aG, kSlab, 1024, kSwz128), make_smem_desc(aG + kTile, kSlab, 1024, kSwz128)};
      bool ok = mbar_wait_warp(bar(KV_FULL), 0, abort_flag) && mbar_wait_warp(bar(Q_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_ss<C>(tS, dK, dQk[0], idesc_ss);  // S^T_0 = K Q^T
        commit_elected(bar(S_FULL));
        ok = mbar_wait_warp(bar(G_FULL), 0, abort_flag);
      }
      if (ok) {
        tc_fence_after_sync();
        issue_ss<C>(tDP, dV, dGk[0], idesc_ss);  // dP^T_0 = V dO^T
        commit_elected(bar(DP_FULL));
      }
      for (int it = 0; ok && it < n_it; ++it) {
        const int s = it & 1, ns = (it + 1) & 1;
        const uint32_t ph = it & 1, nring = ((it + 1) >> 1) & 1;
        if (!mbar_wait_warp(bar(P_FULL), ph, abort_flag)) break;
        tc_fence_after_sync();
        issue_ts<C>(tDV, tS, dGm[s], idesc_ts, it > 0);  // dV += P^T dO
        commit_elected(bar(G_EMPTY + s));
        if (it + 1 < n_it) {
          if (!mbar_wait_warp(bar(Q_FULL + ns), nring, abort_flag)) break;
          tc_fence_after_sync();
          issue_ss<C>(tS, dK, dQk[ns], idesc_ss);  // S^T_{i+1} (after dV_i has read P^T_i)
          commit_elected(bar(S_FULL));
        }
        if (!mbar_wait_warp(bar(DS_FULL), ph, abort_flag)) break;
        tc_fence_after_sync();
        issue_ts<C>(tDK, tDP, dQm[s], idesc_ts, it > 0);  // dK += dS^T Q
        commit_elected(bar(Q_EMPTY + s));
        if (it + 1 < n_it) {
          if (!mbar_wait_warp(bar(G_FULL + ns), nring, abort_flag)) break;
          tc_fence_after_sync();
          issue_ss<C>(tDP, dV, dGk[ns], idesc_ss);  // dP^T_{i+1}
          commit_elected(bar(DP_FULL));
        }
      }
      commit_elected(bar(ACC_FULL));
    }
  } else {
    // compute warps: lanes = keys; warps 0-3 own query columns 0-63, warps 4-7 columns 64-127
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const int tid = threadIdx.x;
    const long long kj = k0 + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int col0 = half * 64;
    const size_t s_base = ((size_t)b * p.H + h) * p.Sq;
    auto fetch_stat = [&](int it) -> float {
      const long long q = (i_begin + it) * BT + (tid & 127);
      if (it >= n_it || q >= (long long)p.Sq) return (tid < 128) ? INFINITY : 0.0f;
      if (tid < 128) {
        const float v = __ldg(p.lse + s_base + q);
        return (v == -INFINITY) ? INFINITY : v * kLog2e;
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
      mbar_arrive(bar(STAT_FULL));
      if (!mbar_wait(bar(STAT_FULL), ph, abort_flag)) { ok = false; break; }
      stat_next = fetch_stat(it + 1);
      const bool need_mask = p.causal && (q0 + p.shift < k0 + (BT - 1));
      const long long cmin_ll = kj - p.shift - q0;  // visible iff column >= cmin
      const int cmin = !need_mask ? 0 : (cmin_ll > BT ? BT : (cmin_ll < 0 ? 0 : (int)cmin_ll));
      if (!mbar_wait(bar(S_FULL), ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      float pr[64];
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + lane_base + col0 + c * 32, r);
        tmem_wait_ld();
        // only a tile on the diagonal has hidden scores: they become -inf here (and 0 below), so that the
        // exponentials of every other tile carry no compare and select
        if (need_mask) {
#pragma unroll
          for (int x = 0; x < 32; ++x)
            if (col0 + c * 32 + x < cmin) r[x] = 0xff800000u;
        }
        // the column statistics are the same for every lane: 128-bit broadcast reads
#pragma unroll
        for (int x4 = 0; x4 < 32; x4 += 4) {
          const float4 l4 = *reinterpret_cast<const float4 *>(lse2 + col0 + c * 32 + x4);
          pr[c * 32 + x4] = ex2_approx(fmaf(__uint_as_float(r[x4]), p.scale_log2, -l4.x));
          pr[c * 32 + x4 + 1] = ex2_approx(fmaf(__uint_as_float(r[x4 + 1]), p.scale_log2, -l4.y));
          pr[c * 32 + x4 + 2] = ex2_approx(fmaf(__uint_as_float(r[x4 + 2]), p.scale_log2, -l4.z));
          pr[c * 32 + x4 + 3] = ex2_approx(fmaf(__uint_as_float(r[x4 + 3]), p.scale_log2, -l4.w));
        }
#pragma unroll
        for (int x = 0; x < 16; ++x) packed[c * 16 + x] = pack2(pr[c * 32 + 2 * x], pr[c * 32 + 2 * x + 1]);
      }
      tmem_st32(tS + lane_base + col0, packed);  // packed P^T over the first half of this thread's own columns
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
        for (int x4 = 0; x4 < 32; x4 += 4) {
          const float4 d4 = *reinterpret_cast<const float4 *>(dlt + col0 + c * 32 + x4);
          packed[c * 16 + x4 / 2] = pack2(pr[c * 32 + x4] * (__uint_as_float(r[x4]) - d4.x),
                                          pr[c * 32 + x4 + 1] * (__uint_as_float(r[x4 + 1]) - d4.y));
          packed[c * 16 + x4 / 2 + 1] = pack2(pr[c * 32 + x4 + 2] * (__uint_as_float(r[x4 + 2]) - d4.z),
                                              pr[c * 32 + x4 + 3] * (__uint_as_float(r[x4 + 3]) - d4.w));
        }
      }
      tmem_st32(tDP + lane_base + col0, packed);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(DS_FULL));
    }
    if (ok && mbar_wait(bar(ACC_FULL), 0, abort_flag)) {
      tc_fence_after_sync();
      // warps 0-3 store dV, warps 4-7 store scale * dK
      const bool row_ok = kj < (long long)p.Sk;
      const float mul = half ? p.scale : 1.0f;
      uint8_t *dst = reinterpret_cast<uint8_t *>(half ? p.dk : p.dv) +
                     (((size_t)b * p.Sk + (size_t)(row_ok ? kj : 0)) * dm + h * HD) * C::kOutElt;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tmem_ld32((half ? tDK : tDV) + lane_base + c * 32, r);
        tmem_wait_ld();
        if (row_ok) {
          if (C::OUT_F32) store_f32x32(dst + c * 128, r, mul);
          else store_bf16x32(dst + c * 64, r, mul);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (warp == 10) {
      commit_elected(bar(DRAIN));  // by the lane that issued the MMAs: the election is deterministic
      for (int n = 0; n < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++n) {
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
// dQ  (a CTA owns 128 queries; TMEM lanes = queries, columns = keys)
// =========================================================================================
namespace dq16 {
enum Bar { QG_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7,   // + ring stage
           S_FULL = 9, S_FREE, DP_FULL, DS_FULL, ACC_FULL, DRAIN, NUM };
template <class C> __host__ __device__ constexpr uint32_t bars_off() { return 6 * C::kTile; }     // Q, dO, K[2], V[2]
template <class C> __host__ __device__ constexpr uint32_t smem_total() { return bars_off<C>() + 256 + 1024; }
}  // namespace dq16

template <class C>
__global__ void __launch_bounds__(kThreads, 1)
k_attn_bwd_dq_bf16(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const Bwd16Params p) {
  using namespace dq16;
  constexpr int HD = C::HD;
  constexpr uint32_t kTile = C::kTile;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aQ = smem_u32(smem), aG = aQ + kTile, aK = aQ + 2 * kTile, aV = aQ + 4 * kTile;  // rings: + stage * kTile
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + bars_off<C>());
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + bars_off<C>() + 160);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + bars_off<C>() + 164);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n_bh = p.B * p.H, bh = blockIdx.x % n_bh;
  const int qt = (int)(gridDim.x / n_bh) - 1 - (int)(blockIdx.x / n_bh);  // heaviest (latest) query tile first
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
        uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.dq) +
                                               (((size_t)b * p.Sq + (size_t)i) * dm + h * HD + (warp >> 2) * (HD / 2)) * C::kOutElt);
#pragma unroll
        for (int x = 0; x < (int)(HD / 2 * C::kOutElt / 16); ++x) dst[x] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    return;
  }

  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM; ++i) mbar_init(bar(i), (i == S_FREE || i == DS_FULL) ? 256 : 1);
    *abort_flag = 0;
    mbar_init_fence();
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
      mbar_arrive_expect_tx(bar(QG_FULL), 2 * kTile);
      for (uint32_t sl = 0; sl < C::kSlabs; ++sl) {
        tma_load_4d(aQ + sl * kSlab, &tmQ, bar(QG_FULL), (int)(sl * 64), (int)h, (int)q0, (int)b);
        tma_load_4d(aG + sl * kSlab, &tmG, bar(QG_FULL), (int)(sl * 64), (int)h, (int)q0, (int)b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1, use = j >> 1;
        if (use > 0 && !mbar_wait(bar(K_EMPTY + s), (use - 1) & 1, abort_flag)) break;
        load_tile<C>(aK + s * kTile, &tmK, bar(K_FULL + s), (int)h, j * BT, (int)b);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1, use = j >> 1;
        if (use > 0 && !mbar_wait(bar(V_EMPTY + s), (use - 1) & 1, abort_flag)) break;
        load_tile<C>(aV + s * kTile, &tmV, bar(V_FULL + s), (int)h, j * BT, (int)b);
      }
    }
  } else if (warp == 10) {
    // The whole warp runs this role, warp-uniformly; one elected lane issues the MMA and commit instructions and
    // every wait returns the same answer in all lanes (see elect_one).
    {
      const uint32_t idesc_ss = make_idesc(kFmtBF16, BT, BT, 0, 0);
      const uint32_t idesc_ts = make_idesc(kFmtBF16, BT, HD, 0, 1);
      const uint64_t dQ = make_smem_desc(aQ, 16, 1024, kSwz128), dG = make_smem_desc(aG, 16, 1024, kSwz128);
      const uint64_t dKk[2] = {make_smem_desc(aK, 16, 1024, kSwz128), make_smem_desc(aK + kTile, 16, 1024, kSwz128)};
      const uint64_t dKm[2] = {make_smem_desc(aK, kSlab, 1024, kSwz128), make_smem_desc(aK + kTile, kSlab, 1024, kSwz128)};
      const uint64_t dVk[2] = {make_smem_desc(aV, 16, 1024, kSwz128), make_smem_desc(aV + kTile, 16, 1024, kSwz128)};
      bool ok = mbar_wait_warp(bar(QG_FULL), 0, abort_flag) && mbar_wait_warp(bar(K_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_ss<C>(tS, dQ, dKk[0], idesc_ss);  // S_0 = Q K^T
        commit_elected(bar(S_FULL));
        ok = mbar_wait_warp(bar(V_FULL), 0, abort_flag);
      }
      if (ok) {
        tc_fence_after_sync();
        issue_ss<C>(tDP, dG, dVk[0], idesc_ss);  // dP_0 = dO V^T
        commit_elected(bar(DP_FULL));
        commit_elected(bar(V_EMPTY));
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int s = j & 1, ns = (j + 1) & 1;
        const uint32_t ph = j & 1, nring = ((j + 1) >> 1) & 1;
        if (j + 1 < n_kv) {
          if (!mbar_wait_warp(bar(S_FREE), ph, abort_flag) || !mbar_wait_warp(bar(K_FULL + ns), nring, abort_flag)) break;
          tc_fence_after_sync();
          issue_ss<C>(tS, dQ, dKk[ns], idesc_ss);  // S_{j+1}: P_j already lives in registers
          commit_elected(bar(S_FULL));
        }
        if (!mbar_wait_warp(bar(DS_FULL), ph, abort_flag)) break;
        tc_fence_after_sync();
        issue_ts<C>(tDQ, tDP, dKm[s], idesc_ts, j > 0);  // dQ += dS K
        commit_elected(bar(K_EMPTY + s));
        if (j + 1 < n_kv) {
          if (!mbar_wait_warp(bar(V_FULL + ns), nring, abort_flag)) break;
          tc_fence_after_sync();
          issue_ss<C>(tDP, dG, dVk[ns], idesc_ss);  // dP_{j+1} (after dQ_j has read dS_j)
          commit_elected(bar(DP_FULL));
          commit_elected(bar(V_EMPTY + ns));
        }
      }
      commit_elected(bar(ACC_FULL));
    }
  } else {
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
        // only the last key tiles of a row have hidden scores: they become -inf here (and 0 below), so that the
        // exponentials of every other tile carry no compare and select
        if (need_mask) {
#pragma unroll
          for (int x = 0; x < 32; ++x)
            if (!(key0 + col0 + c * 32 + x < kmax)) r[x] = 0xff800000u;
        }
#pragma unroll
        for (int x = 0; x < 32; ++x) pr[c * 32 + x] = ex2_approx(fmaf(__uint_as_float(r[x]), p.scale_log2, -lse2));
      }
      tc_fence_before_sync();
      mbar_arrive(bar(S_FREE));
      if (!mbar_wait(bar(DP_FULL), ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tDP + lane_base + col0 + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 16; ++x)
          packed[c * 16 + x] = pack2(pr[c * 32 + 2 * x] * (__uint_as_float(r[2 * x]) - dlt),
                                     pr[c * 32 + 2 * x + 1] * (__uint_as_float(r[2 * x + 1]) - dlt));
      }
      tmem_st32(tDP + lane_base + col0, packed);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(DS_FULL));
    }
    if (ok && mbar_wait(bar(ACC_FULL), 0, abort_flag)) {
      tc_fence_after_sync();
      uint8_t *dst = reinterpret_cast<uint8_t *>(p.dq) +
                     (((size_t)b * p.Sq + (size_t)(row_ok ? i : 0)) * dm + h * HD + half * (HD / 2)) * C::kOutElt;
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {   // each half stores HD/2 dims, 32 at a time
        uint32_t r[32];
        tmem_ld32(tDQ + lane_base + half * (HD / 2) + c * 32, r);
        tmem_wait_ld();
        if (row_ok) {
          if (C::OUT_F32) store_f32x32(dst + c * 128, r, p.scale);
          else store_bf16x32(dst + c * 64, r, p.scale);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (warp == 10) {
      commit_elected(bar(DRAIN));  // by the lane that issued the MMAs: the election is deterministic
      for (int n = 0; n < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++n) {
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

// delta[b][h][i] = sum_d dO * O for bf16 tensors: same streaming pattern as the fp32 pre-pass
// (32 rows x all heads per block, 16-byte loads = 8 bf16, transposed through shared memory).
template <int LPS>  // lanes per (row, head) segment = D / 8
__global__ void __launch_bounds__(256) k_delta_vec_bf16(const uint4 *__restrict__ o, const uint4 *__restrict__ g,
                                                        float *__restrict__ delta, uint32_t H, uint32_t S,
                                                        uint32_t tiles_per_batch) {
  extern __shared__ float s_sum[];  // [H][32]
  const uint32_t b = blockIdx.x / tiles_per_batch;
  const uint32_t i0 = (blockIdx.x % tiles_per_batch) * 32u;
  const uint32_t rows = (S - i0) < 32u ? (S - i0) : 32u;
  const uint32_t nseg = rows * H;
  const size_t chunk = ((size_t)b * S + i0) * H * LPS;
  const uint32_t grp = threadIdx.x / LPS, lane = threadIdx.x % LPS;
  constexpr uint32_t kGroups = 256 / LPS;
  for (uint32_t sg0 = 0; sg0 < nseg; sg0 += kGroups) {
    const uint32_t sg = sg0 + grp;
    float acc = 0.0f;
    if (sg < nseg) {
      const uint4 a = __ldg(o + chunk + (size_t)sg * LPS + lane);
      const uint4 c = __ldg(g + chunk + (size_t)sg * LPS + lane);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        acc = fmaf(__uint_as_float(aw[w] << 16), __uint_as_float(cw[w] << 16), acc);
        acc = fmaf(__uint_as_float(aw[w] & 0xffff0000u), __uint_as_float(cw[w] & 0xffff0000u), acc);
      }
    }
#pragma unroll
    for (int off = LPS / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0 && sg < nseg) s_sum[(sg % H) * 32u + sg / H] = acc;
  }
  __syncthreads();
  for (uint32_t idx = threadIdx.x; idx < 32u * H; idx += 256u) {
    const uint32_t h = idx >> 5, ii = idx & 31u;
    if (ii < rows) delta[((size_t)b * H + h) * S + i0 + ii] = s_sum[idx];
  }
}

template <class C>
int launch_backward(const AttnParams &p, cudaStream_t s) {
  static bool attr_set[64] = {false};
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev)) != DF_OK) return DF_ERR_CUDA;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(k_attn_bwd_dkdv_bf16<C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kv16::smem_total<C>())) != DF_OK ||
        check_cuda(cudaFuncSetAttribute(k_attn_bwd_dq_bf16<C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)dq16::smem_total<C>())) != DF_OK)
      return DF_ERR_CUDA;
    attr_set[dev] = true;
  }
  CUtensorMap tmQ, tmG, tmK, tmV;
  if (!encode_head_tile_map(&tmQ, p.q, true, C::HD, p.B, p.H, p.Sq, BT, false) ||
      !encode_head_tile_map(&tmG, p.d_out, true, C::HD, p.B, p.H, p.Sq, BT, false) ||
      !encode_head_tile_map(&tmK, p.k, true, C::HD, p.B, p.H, p.Sk, BT, false) ||
      !encode_head_tile_map(&tmV, p.v, true, C::HD, p.B, p.H, p.Sk, BT, false)) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  Bwd16Params bp;
  bp.lse = p.lse_in;
  bp.delta = p.delta_in;
  bp.dq = p.d_q;
  bp.dk = p.d_k;
  bp.dv = p.d_v;
  bp.B = p.B; bp.H = p.H; bp.Sq = p.Sq; bp.Sk = p.Sk;
  bp.scale = p.scale;
  bp.scale_log2 = p.scale * kLog2e;
  bp.causal = p.causal;
  bp.shift = p.shift;
  bp.status = device_status_ptr();
  const dim3 grid_kv(((p.Sk + BT - 1) / BT) * p.B * p.H);
  k_attn_bwd_dkdv_bf16<C><<<grid_kv, kThreads, kv16::smem_total<C>(), s>>>(tmK, tmV, tmQ, tmG, bp);
  note_launch();
  if (check_cuda(cudaGetLastError()) != DF_OK) return DF_ERR_CUDA;
  const dim3 grid_q(((p.Sq + BT - 1) / BT) * p.B * p.H);
  k_attn_bwd_dq_bf16<C><<<grid_q, kThreads, dq16::smem_total<C>(), s>>>(tmQ, tmG, tmK, tmV, bp);
  note_launch();
  return check_cuda(cudaGetLastError());
}

}  // namespace

bool tensor_backward_bf16_supported(const AttnParams &p) {
  if (p.Sk == 0 || p.Sq == 0 || p.B == 0 || (p.D != 64 && p.D != 128)) return false;
  if (!(p.scale > 0.0f) || !isfinite(p.scale)) return false;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                         reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.d_out) |
                         reinterpret_cast<uintptr_t>(p.d_q) | reinterpret_cast<uintptr_t>(p.d_k) |
                         reinterpret_cast<uintptr_t>(p.d_v);
  if (bits & 15u) return false;
  if ((uint64_t)p.B * p.H * ((uint64_t)(p.Sq > p.Sk ? p.Sq : p.Sk) / BT + 1) > 0x7fffffffull) return false;
  if ((uint64_t)p.Sq * p.H * p.D * 2 >= (1ull << 40) || (uint64_t)p.Sk * p.H * p.D * 2 >= (1ull << 40)) return false;
  if (p.shift > (1ll << 40) || p.shift < -(1ll << 40)) return false;
  return true;
}

int tensor_backward_bf16(const AttnParams &p, cudaStream_t s) {
  if (p.out_f32) return p.D == 64 ? launch_backward<Cfg16<64, true>>(p, s) : launch_backward<Cfg16<128, true>>(p, s);
  return p.D == 64 ? launch_backward<Cfg16<64>>(p, s) : launch_backward<Cfg16<128>>(p, s);
}

// o_in and d_out are bf16 [B][S][H*D] (D = 64 or 128, 16-byte aligned), delta fp32 [B][H][S].
int delta_prepass_bf16(const AttnParams &p, cudaStream_t s) {
  if (p.Sq == 0 || p.B == 0 || p.H == 0) return DF_OK;
  if ((p.D != 64 && p.D != 128) || p.H > 256) return DF_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(p.o_in) | reinterpret_cast<uintptr_t>(p.d_out)) & 15u) return DF_ERR_UNSUPPORTED;
  const uint32_t tiles = (p.Sq + 31) / 32;
  const dim3 grid(p.B * tiles);
  const size_t smem = (size_t)p.H * 32 * sizeof(float);
  const uint4 *o4 = reinterpret_cast<const uint4 *>(p.o_in);
  const uint4 *g4 = reinterpret_cast<const uint4 *>(p.d_out);
  if (p.D == 64) k_delta_vec_bf16<8><<<grid, 256, smem, s>>>(o4, g4, p.delta, p.H, p.Sq, tiles);
  else k_delta_vec_bf16<16><<<grid, 256, smem, s>>>(o4, g4, p.delta, p.H, p.Sq, tiles);
  note_launch();
  return check_cuda(cudaGetLastError());
}

}  // namespace df
