// attn_fwd_sm100.cu — fused causal attention forward for B200 (sm_100a), fp32 API, TF32 MMA.
//
// Replaces the arithmetic of kernel_fused_mha_fwd_tiled
// (darkforest-cuda/kernels/attention_fused.cu:41-159): O = softmax(scale*QK^T + mask) V per
// head on [S, H*D] tensors, plus the logsumexp the reference does not save.
//
// Structure (one CTA = one 128-row query tile of one (batch, head); two CTAs per SM so that one
// CTA's softmax overlaps the other's MMAs):
//   warp 4      TMA producer: Q once, then K_j / V_j tiles (128 keys x 64 dims, two 128-byte
//               swizzled slabs each) through single K and V buffers, released by MMA commits.
//               The tensor maps are typed TFLOAT32, so the copy engine rounds fp32 to TF32
//               (round to nearest even) on the way in; fed raw fp32 the MMA would truncate 13
//               mantissa bits, which costs about 3x in output error.
//   warp 5      MMA issuer (one thread): S = Q K_j^T (kind::tf32, SS, 128x128x64) into TMEM,
//               then O += P V_j (TS form: P read from TMEM; V is an MN-major 32-bit operand,
//               which must use the 128-byte swizzle with 32-byte atoms)
//   warps 0-3   softmax: one thread per query row reads S from TMEM, masks the diagonal tile,
//               keeps a lazily updated running maximum (O and l are rescaled only when the
//               maximum grew by more than 2^8), writes P = 2^(s*scale*log2e - m) rounded to TF32
//               over S in TMEM, and finally normalises O and stores O and lse
// Causal block skipping: a query tile only visits key tiles that contain a visible key; CTAs
// are ordered heaviest tile first.
//
// Every mbarrier wait is bounded (sm100_ptx.cuh: mbar_wait). If one gives up, the CTA raises
// its abort flag, all roles fall through to the common teardown (drain copies and MMAs, free
// TMEM), and bit 0 of the device status word is set for df_sync_status to report.
#include <math.h>
#include <stdlib.h>

#include "df_common.cuh"
#include "sm100_ptx.cuh"

namespace df {

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

namespace {

using namespace ptx;

constexpr int BM = 128;   // query rows per CTA
constexpr int BN = 128;   // keys per tile
constexpr int HD = 64;    // head dimension of this kernel
constexpr int kFwdThreads = 192;
constexpr uint32_t kSlabBytes = 128 * 128;        // 128 rows x 128 B
constexpr uint32_t kTileBytes = 2 * kSlabBytes;   // 128 x 64 fp32
constexpr uint32_t kTmemCols = 256;               // S/P: 128 columns, O: 64 columns
constexpr float kRescaleThreshold = 8.0f;         // log2 units

struct FwdParams {
  float *out;
  float *lse;
  uint32_t B, H, Sq, Sk;
  float scale_log2;
  int causal;
  long long shift;
  unsigned int *status;
};

enum Bar { Q_FULL = 0, K_FULL, K_EMPTY, V_FULL, V_EMPTY, S_FULL, P_FULL, O_FULL, DRAIN, NUM_BARS };

constexpr uint32_t kSmemBars = 3 * kTileBytes;
constexpr uint32_t kSmemTotal = kSmemBars + 256 + 1024;

__global__ void __launch_bounds__(kFwdThreads, 2)
k_attn_fwd_tf32_d64(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float *sQ = reinterpret_cast<float *>(smem);
  float *sK = reinterpret_cast<float *>(smem + kTileBytes);
  float *sV = reinterpret_cast<float *>(smem + 2 * kTileBytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kSmemBars);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kSmemBars + 128);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + kSmemBars + 132);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;  // heaviest (latest) query tile first
  const uint32_t b = blockIdx.y / p.H, h = blockIdx.y % p.H;
  const long long q0 = (long long)qt * BM;

  long long kv_end = p.causal ? q0 + (BM - 1) + p.shift + 1 : (long long)p.Sk;
  if (kv_end > (long long)p.Sk) kv_end = p.Sk;
  if (kv_end < 0) kv_end = 0;
  const int n_kv = (int)((kv_end + BN - 1) / BN);

  if (n_kv == 0) {
    // no key is visible to any row of this tile: O = 0, lse = -inf
    if (warp < 4) {
      const long long i = q0 + warp * 32 + lane;
      if (i < (long long)p.Sq) {
        float4 *dst = reinterpret_cast<float4 *>(p.out + (((size_t)b * p.Sq + (size_t)i) * p.H + h) * HD);
#pragma unroll
        for (int x = 0; x < HD / 4; ++x) dst[x] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.lse) p.lse[((size_t)b * p.H + h) * p.Sq + (size_t)i] = -INFINITY;
      }
    }
    return;
  }

  auto bar = [&](int id) { return smem_u32(&bars[id]); };

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(K_FULL), 1);
    mbar_init(bar(K_EMPTY), 1);
    mbar_init(bar(V_FULL), 1);
    mbar_init(bar(V_EMPTY), 1);
    mbar_init(bar(S_FULL), 1);
    mbar_init(bar(P_FULL), 128);
    mbar_init(bar(O_FULL), 1);
    mbar_init(bar(DRAIN), 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const uint32_t tS = tmem;        // S and P share these 128 columns
  const uint32_t tO = tmem + 128;  // 64 columns

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(Q_FULL), kTileBytes);
      tma_load_4d(smem_u32(sQ), &tmQ, bar(Q_FULL), 0, (int)h, (int)q0, (int)b);
      tma_load_4d(smem_u32(sQ) + kSlabBytes, &tmQ, bar(Q_FULL), 32, (int)h, (int)q0, (int)b);
      for (int j = 0; j < n_kv; ++j) {
        if (j > 0 && !mbar_wait(bar(K_EMPTY), (j - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(bar(K_FULL), kTileBytes);
        tma_load_4d(smem_u32(sK), &tmK, bar(K_FULL), 0, (int)h, j * BN, (int)b);
        tma_load_4d(smem_u32(sK) + kSlabBytes, &tmK, bar(K_FULL), 32, (int)h, j * BN, (int)b);
        if (j > 0 && !mbar_wait(bar(V_EMPTY), (j - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(bar(V_FULL), kTileBytes);
        tma_load_4d(smem_u32(sV), &tmV, bar(V_FULL), 0, (int)h, j * BN, (int)b);
        tma_load_4d(smem_u32(sV) + kSlabBytes, &tmV, bar(V_FULL), 32, (int)h, j * BN, (int)b);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc(kFmtTF32, BM, BN, 0, 0);
      const uint32_t idesc_pv = make_idesc(kFmtTF32, BM, HD, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag);
      for (int j = 0; ok && j < n_kv; ++j) {
        if (!mbar_wait(bar(K_FULL), j & 1, abort_flag)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < HD / 8; ++kk) {
          const uint32_t off = (kk >> 2) * kSlabBytes + (kk & 3) * 32;
          mma_tf32_ss(tS, make_smem_desc_sw128(aQ + off, 16, 1024), make_smem_desc_sw128(aK + off, 16, 1024),
                      idesc_qk, kk > 0);
        }
        mma_commit(bar(S_FULL));
        mma_commit(bar(K_EMPTY));
        if (!mbar_wait(bar(V_FULL), j & 1, abort_flag)) break;
        if (!mbar_wait(bar(P_FULL), j & 1, abort_flag)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BN / 8; ++kk) {
          mma_tf32_ts(tO, tS + kk * 8, make_smem_desc(aV + kk * 1024, kSlabBytes, 512, kSwz128B32), idesc_pv,
                      (j > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(bar(O_FULL));
        mma_commit(bar(V_EMPTY));
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue
    const int row = warp * 32 + lane;
    const long long i = q0 + row;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    long long kmax_ll = p.causal ? i + p.shift + 1 : (long long)p.Sk;
    if (kmax_ll > (long long)p.Sk) kmax_ll = p.Sk;
    if (kmax_ll < 0) kmax_ll = 0;
    const int kmax = (int)kmax_ll;  // keys [0, kmax) are visible to this row
    float m_run = -INFINITY, m_used = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(bar(S_FULL), j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int key0 = j * BN;
      const bool need_mask = key0 + BN > kmax;
      // pass 1: row maximum of the visible raw scores
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + lane_base + c * 32, r);
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int x = 0; x < 32; ++x)
            mx = fmaxf(mx, (key0 + c * 32 + x < kmax) ? __uint_as_float(r[x]) : -INFINITY);
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) mx = fmaxf(mx, __uint_as_float(r[x]));
        }
      }
      m_run = fmaxf(m_run, mx * p.scale_log2);
      // lazy rescale, decided per warp so that the TMEM accesses stay warp-uniform
      const bool want = (m_run - m_used > kRescaleThreshold) || (m_used == -INFINITY && m_run > -INFINITY);
      if (__any_sync(0xffffffffu, want)) {
        const float alpha = (m_used == -INFINITY) ? 0.0f : ex2_approx(m_used - m_run);
        l *= alpha;
        m_used = m_run;
        if (j > 0) {
          if (!mbar_wait(bar(O_FULL), (j - 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + lane_base + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) r[x] = __float_as_uint(__uint_as_float(r[x]) * alpha);
            tmem_st32(tO + lane_base + c * 32, r);
          }
        }
      }
      const float neg_m = (m_used == -INFINITY) ? 0.0f : -m_used;
      // pass 2: P = 2^(s*scale_log2 - m), rounded to TF32, written over S
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tS + lane_base + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          float e = ex2_approx(fmaf(__uint_as_float(r[x]), p.scale_log2, neg_m));
          if (need_mask && !(key0 + c * 32 + x < kmax)) e = 0.0f;
          const uint32_t pr = cvt_rna_tf32(e);
          l += __uint_as_float(pr);
          r[x] = pr;
        }
        tmem_st32(tS + lane_base + c * 32, r);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(P_FULL));
    }
    if (ok && mbar_wait(bar(O_FULL), (n_kv - 1) & 1, abort_flag)) {
      tc_fence_after_sync();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const bool row_ok = i < (long long)p.Sq;
      float4 *dst = reinterpret_cast<float4 *>(p.out + (((size_t)b * p.Sq + (size_t)(row_ok ? i : 0)) * p.H + h) * HD);
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + lane_base + c * 32, r);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int x = 0; x < 8; ++x)
            dst[c * 8 + x] = make_float4(__uint_as_float(r[4 * x]) * inv, __uint_as_float(r[4 * x + 1]) * inv,
                                         __uint_as_float(r[4 * x + 2]) * inv, __uint_as_float(r[4 * x + 3]) * inv);
        }
      }
      if (row_ok && p.lse)
        p.lse[((size_t)b * p.H + h) * p.Sq + (size_t)i] =
            l > 0.0f ? (m_used + lg2_approx(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  // ---------------------------------------------------------------- teardown (all roles)
  tc_fence_before_sync();
  __syncthreads();
  const bool aborted = *abort_flag != 0u;
  if (aborted) {
    // error path only: give outstanding copies and MMAs a bounded chance to land before the
    // shared and tensor memory of this CTA are released
    if (warp == 5 && lane == 0) {
      mma_commit(bar(DRAIN));
      for (int t = 0; t < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++t) {
      }
    }
    if (warp == 4 && lane == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, DEV_STATUS_WAIT_EXPIRED);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

bool tensor_forward_supported(const AttnParams &p) {
  if (env_flag("DF_ATTN_DISABLE_TENSOR", 0)) return false;  // debugging aid: SIMT kernels only
  if (p.D != HD || p.Sk == 0 || p.Sq == 0 || p.B == 0) return false;
  if (!(p.scale > 0.0f) || !isfinite(p.scale)) return false;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                         reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.out);
  if (bits & 15u) return false;
  if ((uint64_t)p.B * p.H > 65535u) return false;
  if ((uint64_t)p.Sq * p.H * HD * 4 >= (1ull << 40) || (uint64_t)p.Sk * p.H * HD * 4 >= (1ull << 40)) return false;
  if (p.shift > (1ll << 40) || p.shift < -(1ll << 40)) return false;
  return true;
}

int tensor_forward(const AttnParams &p, cudaStream_t s) {
  static bool attr_set[64] = {false};
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev)) != DF_OK) return DF_ERR_CUDA;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(k_attn_fwd_tf32_d64, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kSmemTotal)) != DF_OK)
      return DF_ERR_CUDA;
    attr_set[dev] = true;
  }
  CUtensorMap tmQ, tmK, tmV;
  if (!encode_head_tile_map(&tmQ, p.q, p.B, p.H, p.Sq, BM, false) ||
      !encode_head_tile_map(&tmK, p.k, p.B, p.H, p.Sk, BN, false) ||
      !encode_head_tile_map(&tmV, p.v, p.B, p.H, p.Sk, BN, true)) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  FwdParams fp;
  fp.out = p.out;
  fp.lse = p.lse;
  fp.B = p.B; fp.H = p.H; fp.Sq = p.Sq; fp.Sk = p.Sk;
  fp.scale_log2 = p.scale * 1.4426950408889634f;
  fp.causal = p.causal;
  fp.shift = p.shift;
  fp.status = device_status_ptr();
  const dim3 grid((p.Sq + BM - 1) / BM, p.B * p.H);
  k_attn_fwd_tf32_d64<<<grid, kFwdThreads, kSmemTotal, s>>>(tmQ, tmK, tmV, fp);
  note_launch();
  return check_cuda(cudaGetLastError());
}

}  // namespace df
