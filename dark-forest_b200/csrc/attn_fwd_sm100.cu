// attn_fwd_sm100.cu — fused causal attention forward for B200 (sm_100a), fp32 API, TF32 MMA.
//
// Replaces the arithmetic of kernel_fused_mha_fwd_tiled
// (darkforest-cuda/kernels/attention_fused.cu:41-159): O = softmax(scale*QK^T + mask) V per
// head on [S, H*D] tensors, plus the logsumexp the reference does not save.
//
// Structure: one CTA per SM works on TWO 128-row query tiles (A, B) of one (batch, head) that
// share every K/V tile, so that the tensor pipe runs one tile's MMAs while the other tile is in
// its softmax (measured: two independent CTAs per SM contend for the same unit instead).
//   warp 16     TMA producer: Q_A, Q_B once, then K_j / V_j tiles (128 keys x 64 dims, two
//               128-byte swizzled slabs each) through two-stage K and V rings released by MMA
//               commits. The tensor maps are typed TFLOAT32, so the copy engine rounds fp32 to
//               TF32 (round to nearest even) on the way in; fed raw fp32 the MMA would truncate
//               13 mantissa bits, which costs about 3x in output error.
//   warp 17     MMA issuer (all lanes run the role, elect.sync around the tensor instructions), order
//               PV_A(j) QK_A(j+1) PV_B(j) QK_B(j+1) ...
//               S = Q K_j^T is kind::tf32 SS 128x128x64 into TMEM; O += P V_j is the TS form (P
//               read from TMEM; V is an MN-major 32-bit operand, which must use the 128-byte
//               swizzle with 32-byte atoms). At the pipe's rate a 128x128x8 TF32 MMA takes 64 cycles and
//               a 128x64x8 one 32: ~1.0k cycles of tensor pipe per tile.
//   warps 0-7   softmax of tile A, warps 8-15 of tile B: two threads per query row (64 key
//               columns each) read S from TMEM, mask the diagonal tile, combine their maxima
//               through shared memory, keep a lazily updated running maximum (O and l are rescaled
//               only when the maximum grew by more than 2^8), write P = 2^(s*scale*log2e - m)
//               rounded to TF32 over S in TMEM, and finally normalise O and store O and lse.
// Causal block skipping: a query tile only visits key tiles that contain a visible key; CTAs
// are ordered heaviest first.
//
// Every mbarrier wait is bounded (sm100_ptx.cuh: mbar_wait). If one gives up, the CTA raises
// its abort flag, all roles fall through to the common teardown (drain copies and MMAs, free
// TMEM), and bit 0 of the device status word is set for df_sync_status to report.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <type_traits>

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

constexpr int BM = 128;        // query rows per tile; a CTA owns two tiles
constexpr int BN = 128;        // keys per K/V tile
constexpr int kStages = 2;     // K and V ring depth
constexpr int kFwdThreads = 576;  // warps 0-15 softmax (8 per tile), 16 TMA, 17 MMA
constexpr uint32_t kSlabBytes = 128 * 128;        // 128 rows x 128 B
constexpr uint32_t kTmemCols = 512;               // S/P: 2 x 128 columns, O: 2 x 64 columns
constexpr float kRescaleThreshold = 8.0f;         // log2 units

// Optional phase trace (build with -DDF_ATTN_TRACE): (event id, SM clock) pairs recorded by the
// MMA thread (slot 0) and by lane 0 of the first softmax warp of tile A (slot 1) and tile B
// (slot 2) of the CTA with blockIdx (0,0); the launcher prints them. Compiled out by default.
#ifdef DF_ATTN_TRACE
__device__ unsigned long long g_fwd_trace[3 * 512];
#define DF_TRACE(slot, id)                                            \
  do {                                                                \
    if (trace_on && tr_n < 255) {                                     \
      g_fwd_trace[(slot)*512 + 2 * tr_n] = (id);                      \
      g_fwd_trace[(slot)*512 + 2 * tr_n + 1] = clock64();             \
      ++tr_n;                                                         \
    }                                                                 \
  } while (0)
#else
#define DF_TRACE(slot, id) do { } while (0)
#endif

struct FwdParams {
  void *out;  // fp32 or bf16 elements, see FwdCfg
  float *lse;
  uint32_t B, H, Sq, Sk;
  float scale_log2;
  int causal;
  long long shift;
  unsigned int *status;
#ifdef DF_ATTN_TRACE
  int debug_mode;  // trace builds only (results are wrong when non-zero): 1 = softmax warps skip their work
#endif
};

// barrier indices; the ones followed by "+ stage" / "+ tile" are pairs
enum Bar {
  Q_FULL = 0,
  K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7,                 // + stage
  S_FULL = 9, P_FULL = 11, O_FULL = 13, X_FULL = 15, L_FULL = 17,   // + tile
  DRAIN = 19, NUM_BARS = 20
};

// Compile-time shape of one kernel instance: head dimension and element type of Q/K/V/O.
//   <64, false>  fp32 API, kind::tf32 MMA (rows of 256 B = two 128-byte slabs per tile)
//   <64, true>   bf16 API, kind::f16 MMA  (one slab)      <128, true>  bf16, two slabs
// A K-step of either kind consumes 32 bytes of K per row, so QK takes HD*elt/32 MMAs and PV 128
// keys take 16 (tf32, 8 keys each) or 8 (bf16, 16 keys each) MMAs of N = HD.
template <int HD_, bool BF16_, bool OUT_F32_ = !BF16_>
struct FwdCfg {
  static constexpr int HD = HD_;
  static constexpr bool BF16 = BF16_;
  static constexpr bool OUT_F32 = OUT_F32_;                     // O as fp32 (always for the fp32 API; optional for bf16 inputs:
                                                                // ring partials are merged in fp32)
  static constexpr uint32_t kOutElt = OUT_F32_ ? 4 : 2;
  static constexpr uint32_t kElt = BF16_ ? 2 : 4;
  static constexpr uint32_t kSlabs = HD_ * kElt / 128;
  static constexpr uint32_t kBoxElems = 128 / kElt;             // elements per 128-byte slab row
  static constexpr uint32_t kTileBytes = kSlabs * kSlabBytes;   // 128 rows x HD
  static constexpr uint32_t kSmemK = 2 * kTileBytes;            // after Q_A, Q_B
  static constexpr uint32_t kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr uint32_t kSmemXch = kSmemV + kStages * kTileBytes;  // per tile: max[2][2][128] + l[2][128] floats
  static constexpr uint32_t kSmemBars = kSmemXch + 2 * 768 * 4;
  static constexpr uint32_t kSmemTotal = kSmemBars + 256 + 1024;
  static constexpr uint32_t kFmt = BF16_ ? kFmtBF16 : kFmtTF32;
  static constexpr int kQkSteps = HD_ * kElt / 32;
  static constexpr int kPvSteps = BF16_ ? 8 : 16;
  static constexpr uint32_t kPvStepBytes = BF16_ ? 2048 : 1024;  // 16 or 8 key rows of 128 B
  static constexpr uint32_t kOCols = 256;                       // TMEM column of O_A; O_B follows at + HD
  // When O has the element size of Q, a finished O tile is staged in the shared memory of its Q
  // tile and written by one tiled bulk store; otherwise (fp32 partials of bf16 inputs) every
  // thread stores its half row directly.
  static constexpr bool kStoreViaSmem = (kOutElt == kElt);
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Number of key tiles visible to the 128-row query tile that starts at q0 (0 if q0 >= Sq).
__device__ __forceinline__ int visible_kv_tiles(const FwdParams &p, long long q0) {
  if (q0 >= (long long)p.Sq) return 0;
  long long kv_end = p.causal ? q0 + (BM - 1) + p.shift + 1 : (long long)p.Sk;
  if (kv_end > (long long)p.Sk) kv_end = p.Sk;
  if (kv_end < 0) kv_end = 0;
  return (int)((kv_end + BN - 1) / BN);
}

template <class C>
__global__ void __launch_bounds__(kFwdThreads, 1)
k_attn_fwd(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int HD = C::HD;
  constexpr uint32_t kTileBytes = C::kTileBytes;
  const uint32_t aQ = smem_u32(smem), aK = aQ + C::kSmemK, aV = aQ + C::kSmemV;
  float *sXch = reinterpret_cast<float *>(smem + C::kSmemXch);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::kSmemBars);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + C::kSmemBars + 192);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + C::kSmemBars + 196);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef DF_ATTN_TRACE
  const bool trace_on = blockIdx.x == 0 && lane == 0 && (warp == 17 || warp == 0 || warp == 8);
  int tr_n = 0;
#endif
  DF_TRACE(warp == 17 ? 0 : (warp == 0 ? 1 : 2), 1);  // kernel entry
  // 1-D grid, (batch, head) fastest: all heads' heaviest (latest) pair of query tiles are
  // dispatched first, then the next lighter one, ... (longest-processing-time-first over the GPU)
  const uint32_t n_bh = p.B * p.H, bh = blockIdx.x % n_bh;
  const int pair = (int)(gridDim.x / n_bh) - 1 - (int)(blockIdx.x / n_bh);
  const uint32_t b = bh / p.H, h = bh % p.H;
  // the HD/2 output elements of query row `row` that the thread of column half `half` stores
  auto out_ptr = [&](long long row, int half) -> uint8_t * {
    return reinterpret_cast<uint8_t *>(p.out) +
           ((((size_t)b * p.Sq + (size_t)row) * p.H + h) * HD + (size_t)half * (HD / 2)) * C::kOutElt;
  };
  const long long q0 = (long long)pair * (2 * BM);         // tile A rows q0.., tile B rows q0+128..
  const int n_kv[2] = {visible_kv_tiles(p, q0), visible_kv_tiles(p, q0 + BM)};
  const int n_max = n_kv[0] > n_kv[1] ? n_kv[0] : n_kv[1];

  // Rows that exist but see no key at all: O = 0, lse = -inf (reference guard, attention_fused.cu:104).
  if (warp < 16) {
    const int t = warp >> 3;
    if (n_kv[t] == 0) {
      const long long i = q0 + t * BM + (warp & 3) * 32 + lane;
      if (i < (long long)p.Sq) {
        const int half = (warp >> 2) & 1;
        float4 *dst = reinterpret_cast<float4 *>(out_ptr(i, half));
#pragma unroll
        for (int x = 0; x < (int)(HD / 2 * C::kOutElt / 16); ++x) dst[x] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (half == 0 && p.lse) p.lse[((size_t)b * p.H + h) * p.Sq + (size_t)i] = -INFINITY;
      }
    }
  }
  if (n_max == 0) return;

  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  // K_j and V_j into ring stage j % kStages
  auto load_kv = [&](int j) {
    const int s = j & 1;
    mbar_arrive_expect_tx(bar(K_FULL + s), kTileBytes);
    for (uint32_t sl = 0; sl < C::kSlabs; ++sl)
      tma_load_4d(aK + s * kTileBytes + sl * kSlabBytes, &tmK, bar(K_FULL + s), (int)(sl * C::kBoxElems), (int)h, j * BN, (int)b);
    mbar_arrive_expect_tx(bar(V_FULL + s), kTileBytes);
    for (uint32_t sl = 0; sl < C::kSlabs; ++sl)
      tma_load_4d(aV + s * kTileBytes + sl * kSlabBytes, &tmV, bar(V_FULL + s), (int)(sl * C::kBoxElems), (int)h, j * BN, (int)b);
  };
  if (warp == 16 && lane == 0) {
    // The producer thread initialises the barriers itself and starts the first copies (Q, then
    // as many K/V tiles as the ring holds) before the CTA-wide set-up barrier, so that their
    // latency overlaps the tensor-memory allocation.
    for (int i = 0; i < NUM_BARS; ++i) {
      const bool wide = (i >= P_FULL && i < P_FULL + 2) || (i >= X_FULL && i < X_FULL + 2) || (i >= L_FULL && i < L_FULL + 2);
      mbar_init(bar(i), wide ? 256 : 1);
    }
    *abort_flag = 0;
    mbar_init_fence();
    mbar_arrive_expect_tx(bar(Q_FULL), 2 * kTileBytes);
    for (int t = 0; t < 2; ++t) {
      // rows beyond Sq are zero-filled by the copy engine
      for (uint32_t sl = 0; sl < C::kSlabs; ++sl)
        tma_load_4d(aQ + t * kTileBytes + sl * kSlabBytes, &tmQ, bar(Q_FULL), (int)(sl * C::kBoxElems), (int)h,
                    (int)(q0 + t * BM), (int)b);
    }
    for (int j = 0; j < n_max && j < kStages; ++j) load_kv(j);
  }
  if (warp == 17) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  DF_TRACE(warp == 17 ? 0 : (warp == 0 ? 1 : 2), 2);  // set-up done (barriers, TMEM)
  // TMEM columns: S/P of tile t at [128 t, 128 t + 128), O of tile t at [256 + 64 t, 256 + 64 t + 64)

  if (warp == 16) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // the first kStages tiles were requested during set-up; every later one waits for its slot
      for (int j = kStages; j < n_max; ++j) {
        const int s = j & 1, use = j >> 1;  // ring stage and how often it has been used before
        if (!mbar_wait(bar(K_EMPTY + s), (use - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(bar(K_FULL + s), kTileBytes);
        for (uint32_t sl = 0; sl < C::kSlabs; ++sl)
          tma_load_4d(aK + s * kTileBytes + sl * kSlabBytes, &tmK, bar(K_FULL + s), (int)(sl * C::kBoxElems), (int)h, j * BN, (int)b);
        if (!mbar_wait(bar(V_EMPTY + s), (use - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(bar(V_FULL + s), kTileBytes);
        for (uint32_t sl = 0; sl < C::kSlabs; ++sl)
          tma_load_4d(aV + s * kTileBytes + sl * kSlabBytes, &tmV, bar(V_FULL + s), (int)(sl * C::kBoxElems), (int)h, j * BN, (int)b);
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs this role, warp-uniformly; one elected lane issues the MMA and commit instructions and
    // every wait returns the same answer in all lanes (see elect_one).
    {
      const uint32_t idesc_qk = make_idesc(C::kFmt, BM, BN, 0, 0);
      const uint32_t idesc_pv = make_idesc(C::kFmt, BM, HD, 0, 1);
      bool ok = mbar_wait_warp(bar(Q_FULL), 0, abort_flag);
      DF_TRACE(0, 3);  // Q landed
      // The descriptor low words of every K-step of both Q tiles and both ring stages are computed once; a batch is
      // then issued by one elected lane as nothing but MMA instructions (the issuing warp shares its scheduler with
      // four busy softmax warps, and every other instruction between two MMAs costs the tensor pipe time).
      // V is the MN-major B operand of PV: 32-bit elements need the 32-byte-atom swizzle (4-row groups,
      // SBO 512), 16-bit elements the ordinary 128-byte swizzle (8-row groups, SBO 1024)
      const uint64_t dQ0 = make_smem_desc(aQ, 16, 1024, kSwz128), dK0 = make_smem_desc(aK, 16, 1024, kSwz128);
      const uint64_t dV0 = make_smem_desc(aV, kSlabBytes, C::BF16 ? 1024 : 512, C::BF16 ? kSwz128 : kSwz128B32);
      const uint32_t hiQK = (uint32_t)(dQ0 >> 32), hiV = (uint32_t)(dV0 >> 32);
      uint32_t loQ[2][C::kQkSteps], loK[2][C::kQkSteps], loV[2][C::kPvSteps];
#pragma unroll
      for (int st = 0; st < 2; ++st) {
#pragma unroll
        for (int kk = 0; kk < C::kQkSteps; ++kk) {
          const uint32_t off = (st * kTileBytes + (kk >> 2) * kSlabBytes + (kk & 3) * 32) >> 4;
          loQ[st][kk] = (uint32_t)dQ0 + off;
          loK[st][kk] = (uint32_t)dK0 + off;
        }
#pragma unroll
        for (int kk = 0; kk < C::kPvSteps; ++kk) loV[st][kk] = (uint32_t)dV0 + ((st * kTileBytes + kk * C::kPvStepBytes) >> 4);
      }
      // one batch of QK^T K-steps (elected lane only); TQ, SK select the register sets at compile time
      auto qk_batch = [&](auto tq, auto sk, uint32_t d_tmem) {
        constexpr int TQ = decltype(tq)::value, SK = decltype(sk)::value;
#pragma unroll
        for (int kk = 0; kk < C::kQkSteps; ++kk) {
          if (C::BF16) mma_f16_ss_lohi(d_tmem, loQ[TQ][kk], hiQK, loK[SK][kk], hiQK, idesc_qk, kk > 0 ? 1u : 0u);
          else mma_tf32_ss_lohi(d_tmem, loQ[TQ][kk], hiQK, loK[SK][kk], hiQK, idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      auto pv_batch = [&](auto sv, uint32_t d_tmem, uint32_t a_tmem, uint32_t acc0) {
        constexpr int SV = decltype(sv)::value;
#pragma unroll
        for (int kk = 0; kk < C::kPvSteps; ++kk) {
          if (C::BF16) mma_f16_ts_lohi(d_tmem, a_tmem + kk * 8, loV[SV][kk], hiV, idesc_pv, kk > 0 ? 1u : acc0);
          else mma_tf32_ts_lohi(d_tmem, a_tmem + kk * 8, loV[SV][kk], hiV, idesc_pv, kk > 0 ? 1u : acc0);
        }
      };
      using I0 = std::integral_constant<int, 0>;
      using I1 = std::integral_constant<int, 1>;
      // bf16 at head dimension 128 keeps the other form (an election and an address add per MMA): its MMAs are twice as
      // long, the precomputed words made the kernel spill, and it measured 2 % slower with them (TF32: 8-11 % faster
      // at S >= 32768, bf16 at head dimension 64: 4 % faster)
      constexpr bool kPure = !(C::BF16 && HD == 128);
      const uint64_t dQ1 = dQ0 + (uint64_t)(kTileBytes >> 4), dK1 = dK0 + (uint64_t)(kTileBytes >> 4), dV1 = dV0 + (uint64_t)(kTileBytes >> 4);
      // S_t = Q_t K_j^T. The last tile to use K_j releases its ring slot.
      auto issue_qk = [&](int t, int j) -> bool {
        const int s = j & 1;
        // tile B reuses the K tile that tile A's product has just waited for (same thread, same phase)
        if ((t == 0 || j >= n_kv[0]) && !mbar_wait_warp(bar(K_FULL + s), (j >> 1) & 1, abort_flag)) return false;
        DF_TRACE(0, 10 + t);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + t * 128;
        const int last_user = (j < n_kv[1]) ? 1 : 0;
        if constexpr (kPure) {
          if (elect_one()) {
            if (t == 0) { if (s) qk_batch(I0{}, I1{}, d_tmem); else qk_batch(I0{}, I0{}, d_tmem); }
            else        { if (s) qk_batch(I1{}, I1{}, d_tmem); else qk_batch(I1{}, I0{}, d_tmem); }
            mma_commit(bar(S_FULL + t));
            if (t == last_user) mma_commit(bar(K_EMPTY + s));
          }
          __syncwarp();
        } else {
          const uint64_t da = t ? dQ1 : dQ0, db = s ? dK1 : dK0;
#pragma unroll
          for (int kk = 0; kk < C::kQkSteps; ++kk) {
            const uint64_t off = (uint64_t)(((kk >> 2) * kSlabBytes + (kk & 3) * 32) >> 4);
            if (elect_one()) mma_f16_ss(d_tmem, da + off, db + off, idesc_qk, kk > 0);
          }
          commit_elected(bar(S_FULL + t));
          if (t == last_user) commit_elected(bar(K_EMPTY + s));
        }
        DF_TRACE(0, 12 + t);
        return true;
      };
      // O_t += P_t V_j
      auto issue_pv = [&](int t, int j) -> bool {
        const int s = j & 1;
        DF_TRACE(0, 30 + t);
        if ((t == 0 || j >= n_kv[0]) && !mbar_wait_warp(bar(V_FULL + s), (j >> 1) & 1, abort_flag)) return false;
        DF_TRACE(0, 14 + t);
        if (!mbar_wait_warp(bar(P_FULL + t), j & 1, abort_flag)) return false;
        DF_TRACE(0, 16 + t);
        tc_fence_after_sync();
        // P occupies 8 TMEM columns per K-step in both kinds (8 tf32 values, or 16 packed bf16 values)
        const uint32_t d_tmem = tmem + C::kOCols + t * HD, a_tmem = tmem + t * 128;
        const int last_user = (j < n_kv[1]) ? 1 : 0;
        if constexpr (kPure) {
          if (elect_one()) {
            if (s) pv_batch(I1{}, d_tmem, a_tmem, j > 0 ? 1u : 0u); else pv_batch(I0{}, d_tmem, a_tmem, j > 0 ? 1u : 0u);
            mma_commit(bar(O_FULL + t));
            if (t == last_user) mma_commit(bar(V_EMPTY + s));
          }
          __syncwarp();
        } else {
          const uint64_t db = s ? dV1 : dV0;
#pragma unroll
          for (int kk = 0; kk < C::kPvSteps; ++kk) {
            const uint64_t bd = db + (uint64_t)(kk * (C::kPvStepBytes >> 4));
            if (elect_one()) mma_f16_ts(d_tmem, a_tmem + kk * 8, bd, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          }
          commit_elected(bar(O_FULL + t));
          if (t == last_user) commit_elected(bar(V_EMPTY + s));
        }
        DF_TRACE(0, 18 + t);
        return true;
      };
      if (ok && n_kv[0] > 0) ok = issue_qk(0, 0);
      if (ok && n_kv[1] > 0) ok = issue_qk(1, 0);
      for (int j = 0; ok && j < n_max; ++j) {
        for (int t = 0; ok && t < 2; ++t) {
          if (j < n_kv[t]) {
            ok = issue_pv(t, j);
            if (ok && j + 1 < n_kv[t]) ok = issue_qk(t, j + 1);  // overwrites P_t(j) after PV_t(j) has read it
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue
    // Warps 0-7 serve tile A, 8-15 tile B. Within a tile two warpgroups share every query row:
    // warps 0-3 own key columns 0-63 of the K/V tile, warps 4-7 columns 64-127 (a warp reads TMEM
    // lanes 32*(w%4)..+31). The row maximum is combined with the partner thread through shared
    // memory, after which both take identical rescale decisions.
    const int t = warp >> 3;
    const int quarter = warp & 3, half = (warp >> 2) & 1;
    const int row = quarter * 32 + lane;
    const long long i = q0 + t * BM + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + t * 128, tO = tmem + C::kOCols + t * HD;
    const int col0 = half * 64;
    const int nkv = n_kv[t];
    float *xch = sXch + t * 768;
    long long kmax_ll = p.causal ? i + p.shift + 1 : (long long)p.Sk;
    if (kmax_ll > (long long)p.Sk) kmax_ll = p.Sk;
    if (kmax_ll < 0) kmax_ll = 0;
    const int kmax = (int)kmax_ll;  // keys [0, kmax) are visible to this row
    float m_run = -INFINITY, m_used = -INFINITY;
    float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
    bool ok = nkv > 0;
    for (int j = 0; j < nkv; ++j) {
      DF_TRACE(1 + t, 20);
      if (!mbar_wait(bar(S_FULL + t), j & 1, abort_flag)) { ok = false; break; }
      DF_TRACE(1 + t, 21);
      tc_fence_after_sync();
#ifdef DF_ATTN_TRACE
      if (p.debug_mode == 1) {
        tc_fence_before_sync();
        mbar_arrive(bar(P_FULL + t));
        continue;
      }
#endif
      const int key0 = j * BN + col0;
      const bool need_mask = key0 + 64 > kmax;
      // single pass: the thread's 64 scores stay in registers from the maximum to the exponentials
      uint32_t ra[32], rb[32];
      tmem_ld32(tS + lane_base + col0, ra);
      tmem_ld32(tS + lane_base + col0 + 32, rb);
      tmem_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          if (!(key0 + x < kmax)) ra[x] = 0xff800000u;  // -inf: exponentiates to 0
          if (!(key0 + 32 + x < kmax)) rb[x] = 0xff800000u;
        }
      }
      float mx_half;
      {
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int x = 0; x < 32; x += 4) {
          mx0 = fmaxf(mx0, fmaxf(__uint_as_float(ra[x]), __uint_as_float(rb[x])));
          mx1 = fmaxf(mx1, fmaxf(__uint_as_float(ra[x + 1]), __uint_as_float(rb[x + 1])));
          mx2 = fmaxf(mx2, fmaxf(__uint_as_float(ra[x + 2]), __uint_as_float(rb[x + 2])));
          mx3 = fmaxf(mx3, fmaxf(__uint_as_float(ra[x + 3]), __uint_as_float(rb[x + 3])));
        }
        mx_half = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      }
      // exchange the half-row maxima (double-buffered by tile parity)
      DF_TRACE(1 + t, 22);
      float *xmax = xch + (j & 1) * 256;
      xmax[half * 128 + row] = mx_half;
      mbar_arrive(bar(X_FULL + t));
      if (!mbar_wait(bar(X_FULL + t), j & 1, abort_flag)) { ok = false; break; }
      DF_TRACE(1 + t, 23);
      const float mx = fmaxf(mx_half, xmax[(half ^ 1) * 128 + row]);
      m_run = fmaxf(m_run, mx * p.scale_log2);
      // lazy rescale, decided per warp so that the TMEM accesses stay warp-uniform; the partner
      // warp sees the same rows and the same maxima, hence takes the same decision
      const bool want = (m_run - m_used > kRescaleThreshold) || (m_used == -INFINITY && m_run > -INFINITY);
      if (__any_sync(0xffffffffu, want)) {
        const float alpha = (m_used == -INFINITY) ? 0.0f : ex2_approx(m_used - m_run);
        l0 *= alpha; l1 *= alpha; l2 *= alpha; l3 *= alpha;
        m_used = m_run;
        if (j > 0) {
          if (!mbar_wait(bar(O_FULL + t), (j - 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          // each half rescales HD/2 of the O columns, 16 at a time to stay within the register budget
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t ro[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(ro[0]), "=r"(ro[1]), "=r"(ro[2]), "=r"(ro[3]), "=r"(ro[4]), "=r"(ro[5]), "=r"(ro[6]), "=r"(ro[7]),
                  "=r"(ro[8]), "=r"(ro[9]), "=r"(ro[10]), "=r"(ro[11]), "=r"(ro[12]), "=r"(ro[13]), "=r"(ro[14]), "=r"(ro[15])
                : "r"(tO + lane_base + half * (HD / 2) + c * 16)
                : "memory");
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 16; ++x) ro[x] = __float_as_uint(__uint_as_float(ro[x]) * alpha);
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                ::"r"(tO + lane_base + half * (HD / 2) + c * 16), "r"(ro[0]), "r"(ro[1]), "r"(ro[2]), "r"(ro[3]), "r"(ro[4]), "r"(ro[5]),
                  "r"(ro[6]), "r"(ro[7]), "r"(ro[8]), "r"(ro[9]), "r"(ro[10]), "r"(ro[11]), "r"(ro[12]), "r"(ro[13]), "r"(ro[14]),
                  "r"(ro[15])
                : "memory");
          }
        }
      }
      const float neg_m = (m_used == -INFINITY) ? 0.0f : -m_used;
      // P = 2^(s*scale_log2 - m), written over S: TF32-rounded words, or packed bf16 pairs (keys
      // 2c, 2c+1 in TMEM column c; every thread of the row loaded its scores before the exchange
      // barrier above, so overwriting the partner's S columns is safe)
      DF_TRACE(1 + t, 24);
#pragma unroll
      for (int x = 0; x < 32; x += 4) {
        const float e0 = ex2_approx(fmaf(__uint_as_float(ra[x]), p.scale_log2, neg_m));
        const float e1 = ex2_approx(fmaf(__uint_as_float(ra[x + 1]), p.scale_log2, neg_m));
        const float e2 = ex2_approx(fmaf(__uint_as_float(ra[x + 2]), p.scale_log2, neg_m));
        const float e3 = ex2_approx(fmaf(__uint_as_float(ra[x + 3]), p.scale_log2, neg_m));
        if (C::BF16) {
          ra[x / 2] = pack_bf16x2(e0, e1);
          ra[x / 2 + 1] = pack_bf16x2(e2, e3);
          l0 += e0; l1 += e1; l2 += e2; l3 += e3;
        } else {
          // half a TF32 ulp added for the MMA, which drops the low mantissa bits; the row sum takes the unrounded values
          ra[x] = tf32_rna_operand(e0); ra[x + 1] = tf32_rna_operand(e1);
          ra[x + 2] = tf32_rna_operand(e2); ra[x + 3] = tf32_rna_operand(e3);
          l0 += e0; l1 += e1; l2 += e2; l3 += e3;
        }
      }
      if (!C::BF16) tmem_st32(tS + lane_base + col0, ra);
#pragma unroll
      for (int x = 0; x < 32; x += 4) {
        const float e0 = ex2_approx(fmaf(__uint_as_float(rb[x]), p.scale_log2, neg_m));
        const float e1 = ex2_approx(fmaf(__uint_as_float(rb[x + 1]), p.scale_log2, neg_m));
        const float e2 = ex2_approx(fmaf(__uint_as_float(rb[x + 2]), p.scale_log2, neg_m));
        const float e3 = ex2_approx(fmaf(__uint_as_float(rb[x + 3]), p.scale_log2, neg_m));
        if (C::BF16) {
          ra[16 + x / 2] = pack_bf16x2(e0, e1);   // ra[0..15] hold this thread's first 32 keys
          ra[16 + x / 2 + 1] = pack_bf16x2(e2, e3);
          l0 += e0; l1 += e1; l2 += e2; l3 += e3;
        } else {
          // half a TF32 ulp added for the MMA, which drops the low mantissa bits; the row sum takes the unrounded values
          rb[x] = tf32_rna_operand(e0); rb[x + 1] = tf32_rna_operand(e1);
          rb[x + 2] = tf32_rna_operand(e2); rb[x + 3] = tf32_rna_operand(e3);
          l0 += e0; l1 += e1; l2 += e2; l3 += e3;
        }
      }
      if (C::BF16) tmem_st32(tS + lane_base + half * 32, ra);
      else tmem_st32(tS + lane_base + col0 + 32, rb);
      DF_TRACE(1 + t, 25);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(P_FULL + t));
      DF_TRACE(1 + t, 26);
    }
    // combine the two half-row sums, then normalise and store 32 of the 64 output columns each
    float l = (l0 + l1) + (l2 + l3);
    if (ok) {
      float *xl = xch + 512;
      xl[half * 128 + row] = l;
      mbar_arrive(bar(L_FULL + t));
      if (!mbar_wait(bar(L_FULL + t), 0, abort_flag)) ok = false;
      else l += xl[(half ^ 1) * 128 + row];
    }
    if (ok && mbar_wait(bar(O_FULL + t), (nkv - 1) & 1, abort_flag)) {
      tc_fence_after_sync();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const bool row_ok = i < (long long)p.Sq;
      uint8_t *dst = out_ptr(row_ok ? i : 0, half);
      // staging address of this thread's half row inside the (no longer needed) Q tile: the
      // 128-byte swizzle of the store's tensor map puts 16-byte chunk c of row r at c ^ (r % 8)
      constexpr uint32_t kHalfBytes = HD / 2 * C::kOutElt;
      const uint32_t st_off = (uint32_t)half * kHalfBytes;
      uint8_t *stage = smem + t * kTileBytes + (st_off / 128) * kSlabBytes + row * 128;
      const uint32_t chunk0 = (st_off % 128) / 16;
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {   // 32 O columns per step
        uint32_t ro[32];
        tmem_ld32(tO + lane_base + half * (HD / 2) + c * 32, ro);
        tmem_wait_ld();
        if (C::kStoreViaSmem) {
          if (!C::OUT_F32) {
#pragma unroll
            for (int x = 0; x < 4; ++x)
              *reinterpret_cast<uint4 *>(stage + (((chunk0 + c * 4 + x) ^ (row & 7)) << 4)) =
                  make_uint4(pack_bf16x2(__uint_as_float(ro[8 * x]) * inv, __uint_as_float(ro[8 * x + 1]) * inv),
                             pack_bf16x2(__uint_as_float(ro[8 * x + 2]) * inv, __uint_as_float(ro[8 * x + 3]) * inv),
                             pack_bf16x2(__uint_as_float(ro[8 * x + 4]) * inv, __uint_as_float(ro[8 * x + 5]) * inv),
                             pack_bf16x2(__uint_as_float(ro[8 * x + 6]) * inv, __uint_as_float(ro[8 * x + 7]) * inv));
          } else {
#pragma unroll
            for (int x = 0; x < 8; ++x)
              *reinterpret_cast<float4 *>(stage + (((chunk0 + c * 8 + x) ^ (row & 7)) << 4)) =
                  make_float4(__uint_as_float(ro[4 * x]) * inv, __uint_as_float(ro[4 * x + 1]) * inv,
                              __uint_as_float(ro[4 * x + 2]) * inv, __uint_as_float(ro[4 * x + 3]) * inv);
          }
        } else if (row_ok) {
          if (!C::OUT_F32) {
            uint4 *d4 = reinterpret_cast<uint4 *>(dst + c * 64);
#pragma unroll
            for (int x = 0; x < 4; ++x)
              d4[x] = make_uint4(pack_bf16x2(__uint_as_float(ro[8 * x]) * inv, __uint_as_float(ro[8 * x + 1]) * inv),
                                 pack_bf16x2(__uint_as_float(ro[8 * x + 2]) * inv, __uint_as_float(ro[8 * x + 3]) * inv),
                                 pack_bf16x2(__uint_as_float(ro[8 * x + 4]) * inv, __uint_as_float(ro[8 * x + 5]) * inv),
                                 pack_bf16x2(__uint_as_float(ro[8 * x + 6]) * inv, __uint_as_float(ro[8 * x + 7]) * inv));
          } else {
            float4 *d4 = reinterpret_cast<float4 *>(dst + c * 128);
#pragma unroll
            for (int x = 0; x < 8; ++x)
              d4[x] = make_float4(__uint_as_float(ro[4 * x]) * inv, __uint_as_float(ro[4 * x + 1]) * inv,
                                  __uint_as_float(ro[4 * x + 2]) * inv, __uint_as_float(ro[4 * x + 3]) * inv);
          }
        }
      }
      if (row_ok) {
        if (half == 0 && p.lse)
          p.lse[((size_t)b * p.H + h) * p.Sq + (size_t)i] =
              l > 0.0f ? (m_used + lg2_approx(l)) * 0.6931471805599453f : -INFINITY;
      }
      if (C::kStoreViaSmem) {
        // all 256 threads of the tile have staged their rows (second phase of the tile's
        // row-sum barrier); one thread then hands the tile to the copy engine, which drops rows
        // beyond Sq
        fence_proxy_async_smem();
        mbar_arrive(bar(L_FULL + t));
        if ((warp & 7) == 0 && lane == 0 && mbar_wait(bar(L_FULL + t), 1, abort_flag)) {
          for (uint32_t sl = 0; sl < C::kSlabs; ++sl)
            tma_store_4d(&tmO, aQ + t * kTileBytes + sl * kSlabBytes, (int)(sl * C::kBoxElems), (int)h,
                         (int)(q0 + t * BM), (int)b);
          tma_store_commit();
          tma_store_wait_read_all();
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown (all roles)
  DF_TRACE(warp == 17 ? 0 : (warp == 0 ? 1 : 2), 4);  // role finished
  tc_fence_before_sync();
  __syncthreads();
  DF_TRACE(warp == 17 ? 0 : (warp == 0 ? 1 : 2), 5);  // all roles finished
  if (*abort_flag != 0u) {
    // error path only: give outstanding copies and MMAs a bounded chance to land before the
    // shared and tensor memory of this CTA are released
    if (warp == 17) {
      commit_elected(bar(DRAIN));  // by the lane that issued the MMAs: the election is deterministic
      for (int n = 0; n < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++n) {
      }
    }
    if (warp == 16 && lane == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, DEV_STATUS_WAIT_EXPIRED);
    __syncthreads();
  }
  if (warp == 17) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
    DF_TRACE(0, 6);  // TMEM released
  }
}

}  // namespace

bool tensor_forward_supported(const AttnParams &p) {
  if (option(DF_OPT_DISABLE_TENSOR) == 1) return false;  // debugging aid: SIMT kernels only
  if (p.Sk == 0 || p.Sq == 0 || p.B == 0) return false;
  if (p.bf16 ? (p.D != 64 && p.D != 128) : (p.D != 64)) return false;
  if (!(p.scale > 0.0f) || !isfinite(p.scale)) return false;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) |
                         reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.out);
  if (bits & 15u) return false;
  if ((uint64_t)p.B * p.H * ((p.Sq + 2 * BM - 1) / (2 * BM)) > 0x7fffffffull) return false;
  if ((uint64_t)p.Sq * p.H * p.D * 4 >= (1ull << 40) || (uint64_t)p.Sk * p.H * p.D * 4 >= (1ull << 40)) return false;
  if (p.shift > (1ll << 40) || p.shift < -(1ll << 40)) return false;
  return true;
}

namespace {
template <class C>
int launch_forward(const AttnParams &p, cudaStream_t s) {
  static bool attr_set[64] = {false};
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev)) != DF_OK) return DF_ERR_CUDA;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(k_attn_fwd<C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)C::kSmemTotal)) != DF_OK)
      return DF_ERR_CUDA;
    attr_set[dev] = true;
  }
  CUtensorMap tmQ, tmK, tmV, tmO;
  // V is an MN-major operand: 32-bit elements need the 32-byte-atom swizzle, 16-bit ones do not
  if (!encode_head_tile_map(&tmQ, p.q, C::BF16, C::HD, p.B, p.H, p.Sq, BM, false) ||
      !encode_head_tile_map(&tmK, p.k, C::BF16, C::HD, p.B, p.H, p.Sk, BN, false) ||
      !encode_head_tile_map(&tmV, p.v, C::BF16, C::HD, p.B, p.H, p.Sk, BN, !C::BF16) ||
      !encode_head_tile_map(&tmO, C::kStoreViaSmem ? p.out : p.q, C::BF16, C::HD, p.B, p.H, p.Sq, BM, false, true)) {
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
#ifdef DF_ATTN_TRACE
  fp.debug_mode = getenv("DF_ATTN_FWD_DEBUG") ? atoi(getenv("DF_ATTN_FWD_DEBUG")) : 0;
#endif
  const dim3 grid(((p.Sq + 2 * BM - 1) / (2 * BM)) * p.B * p.H);
  k_attn_fwd<C><<<grid, kFwdThreads, C::kSmemTotal, s>>>(tmQ, tmK, tmV, tmO, fp);
  note_launch();
#ifdef DF_ATTN_TRACE
  if (getenv("DF_ATTN_TRACE_DUMP")) {
    static unsigned long long host[3 * 512];
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(host, g_fwd_trace, sizeof(host));
    for (int slot = 0; slot < 3; ++slot)
      for (int e = 0; e < 100; ++e)
        if (host[slot * 512 + 2 * e + 1])
          printf("trace slot %d ev %llu t %llu\n", slot, host[slot * 512 + 2 * e], host[slot * 512 + 2 * e + 1] - host[1]);
  }
#endif
  return check_cuda(cudaGetLastError());
}
}  // namespace

int tensor_forward(const AttnParams &p, cudaStream_t s) {
  if (tensor_forward_persistent_supported(p)) return tensor_forward_persistent(p, s);
  if (!p.bf16) return launch_forward<FwdCfg<64, false>>(p, s);
  if (p.out_f32) return p.D == 64 ? launch_forward<FwdCfg<64, true, true>>(p, s) : launch_forward<FwdCfg<128, true, true>>(p, s);
  return p.D == 64 ? launch_forward<FwdCfg<64, true>>(p, s) : launch_forward<FwdCfg<128, true>>(p, s);
}

}  // namespace df
