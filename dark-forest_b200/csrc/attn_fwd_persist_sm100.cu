// attn_fwd_persist_sm100.cu — persistent fused causal attention forward for B200 (sm_100a),
// fp32 API, TF32 MMA, head dimension 64, whole sequences (Sq == Sk, no causal shift).
//
// Same arithmetic and the same two-query-tiles-per-CTA pipeline as attn_fwd_sm100.cu (which keeps
// serving key blocks with a causal shift, ragged Sq != Sk and the bf16 variants), replacing
// kernel_fused_mha_fwd_tiled (darkforest-cuda/kernels/attention_fused.cu:41-159). What differs:
//   * The grid has at most one CTA per SM. Every CTA walks a static list of work items (a pair
//     of 128-row query tiles of one head), numbered heaviest first and dealt in rounds with odd
//     rounds reversed, and runs them as ONE pipeline: the K/V ring, all barrier phases and the
//     MMA order continue across items, so the next item's K/V tiles, its Q tiles and its first
//     QK^T products are under way while the current item's last PV products finish and its output
//     tiles are stored. Set-up (barriers, tensor-memory allocation) is paid once per SM.
//   * Q lives in tensor memory. A Q tile lands in a 32 KB shared-memory buffer through the
//     TFLOAT32 tensor map (rounded to TF32 in flight), the tile's softmax threads copy their rows
//     into 64 spare TMEM columns, and S = Q K^T is issued in the TS form (A from TMEM). That
//     halves the shared-memory traffic of the QK^T product and frees the buffer: it receives the
//     next item's Q tile while the current item computes and stages the finished O tile for its
//     bulk store in between.
// TMEM columns: S/P of tile t at [128 t, 128 t + 128), O of tile t at [256 + 64 t, +64), Q of
// tile t at [384 + 64 t, +64) = all 512.
//
// Roles: warps 0-7 softmax + epilogue of tile slot A, 8-15 of slot B (two threads per query row),
// warp 16 TMA producer, warp 17 MMA issuer. Every mbarrier wait is bounded (sm100_ptx.cuh).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "df_common.cuh"
#include "sm100_ptx.cuh"

namespace df {
namespace {

using namespace ptx;

constexpr int BM = 128;            // query rows per tile; an item is two tiles
constexpr int BN = 128;            // keys per K/V tile
constexpr int HD = 64;
// HALVES threads share a query row (each owns 128 / HALVES key columns of a step): 2 = sixteen softmax warps, the
// row maximum and sum combined through shared memory; 1 = eight softmax warps, a thread per row, nothing to combine.
// Measured on the B200 with the same inputs: one thread per row (168 registers, two softmax warps per scheduler) is
// 4-5 % slower (S = 16384: 0.86 ms against 0.82 ms), so two threads per row stay the default.
#ifndef DF_FWD_HALVES
#define DF_FWD_HALVES 2
#endif
constexpr int kThreadsOf(int halves) { return (8 * halves + 2) * 32; }
constexpr uint32_t kSlab = 128 * 128;   // 128 rows x 128 B
constexpr uint32_t kTile = 2 * kSlab;   // 128 rows x 64 fp32
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

constexpr uint32_t kSmemLand = 0;                 // Q landing / O staging, one tile per slot
constexpr uint32_t kSmemK = 2 * kTile;            // two ring stages
constexpr uint32_t kSmemV = 4 * kTile;
constexpr uint32_t kSmemXch = 6 * kTile;          // per slot: max[2][2][128] + l[2][128] floats
constexpr uint32_t kSmemBars = kSmemXch + 2 * 768 * 4;
constexpr uint32_t kSmemTotal = kSmemBars + 256 + 1024;

// barrier indices; "+ stage" / "+ slot" mark pairs
enum Bar {
  K_FULL = 0, K_EMPTY = 2, V_FULL = 4, V_EMPTY = 6,                      // + stage
  QL_FULL = 8, QT_FULL = 10, LAND_FREE = 12,                             // + slot: Q landed / Q in TMEM / buffer reusable
  S_FULL = 14, P_FULL = 16, O_FULL = 18, X_FULL = 20, L_FULL = 22,       // + slot
  DRAIN = 24, NUM_BARS = 25
};

struct PParams {
  float *out;
  float *lse;
  uint32_t B, H, S;
  float scale_log2;
  int causal;
  int n_items, n_pairs;
  unsigned int *status;
};

struct Item {
  uint32_t b, h;
  long long q0;   // first row of tile A; tile B starts at q0 + 128
  int n_kv[2];    // key tiles that tile A / B visit; n_kv[1] >= n_kv[0] >= 1
  int n_max;
};

__host__ __device__ __forceinline__ int visible_tiles(const PParams &p, long long q0) {
  if (q0 >= (long long)p.S) return 0;
  long long kv_end = p.causal ? q0 + BM : (long long)p.S;
  if (kv_end > (long long)p.S) kv_end = p.S;
  return (int)((kv_end + BN - 1) / BN);
}
// Item number idx (heaviest first, (batch, head) fastest) -> its head, rows and key-tile counts.
__host__ __device__ __forceinline__ void decode_item(const PParams &p, long long idx, Item *it) {
  const uint32_t n_bh = p.B * p.H, bh = (uint32_t)idx % n_bh;
  it->b = bh / p.H;
  it->h = bh % p.H;
  it->q0 = (long long)(p.n_pairs - 1 - (int)((uint32_t)idx / n_bh)) * (2 * BM);  // latest pair first: most key tiles
  it->n_kv[0] = visible_tiles(p, it->q0);
  // A tile B that lies wholly beyond the sequence runs along on zero-filled queries (nothing of it
  // is stored): both slots then do the same thing in every item, which keeps the pipeline uniform.
  it->n_kv[1] = (it->q0 + BM < (long long)p.S) ? visible_tiles(p, it->q0 + BM) : it->n_kv[0];
  it->n_max = it->n_kv[1];
}
// Item of round r for this CTA (explicit work list, or the snake order); false when the list is exhausted.
__device__ __forceinline__ bool item_of_round(const PParams &p, const SchedTable *tab, int r, Item *it) {
  const long long idx = sched_item(*tab, r, (int)gridDim.x, (int)blockIdx.x, p.n_items);
  if (idx < 0) return false;
  decode_item(p, idx, it);
  return true;
}

#ifdef DF_ATTN_TRACE
__device__ unsigned long long g_pfwd_trace[3 * 1024];
#define DF_PTRACE(slot, id)                                           \
  do {                                                                \
    if (trace_on && tr_n < 511) {                                     \
      g_pfwd_trace[(slot)*1024 + 2 * tr_n] = (id);                    \
      g_pfwd_trace[(slot)*1024 + 2 * tr_n + 1] = clock64();           \
      ++tr_n;                                                         \
    }                                                                 \
  } while (0)
#else
#define DF_PTRACE(slot, id) do { } while (0)
#endif

// INLINE_WAIT: the bounded-wait loop inline at every wait site (faster for short sequences) or one out-of-line
// copy (faster from a few thousand rows on); the launcher picks by sequence length.
template <bool INLINE_WAIT, int HALVES>
__global__ void __launch_bounds__(kThreadsOf(HALVES), 1)
k_attn_fwd_persist_tf32_d64(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                            const __grid_constant__ SchedTable tab, const PParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aL = smem_u32(smem), aK = aL + kSmemK, aV = aL + kSmemV;
  float *sXch = reinterpret_cast<float *>(smem + kSmemXch);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kSmemBars);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kSmemBars + 224);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + kSmemBars + 228);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kSlotWarps = 4 * HALVES;                 // softmax warps per slot
  constexpr int kWarpLoad = 8 * HALVES, kWarpMma = 8 * HALVES + 1;
  constexpr int kSlotThreads = 128 * HALVES;
#ifdef DF_ATTN_TRACE
  const bool trace_on = blockIdx.x == 0 && lane == 0 && (warp == kWarpMma || warp == 0 || warp == kSlotWarps);
  int tr_n = 0;
#endif
  DF_PTRACE(warp == kWarpMma ? 0 : (warp == 0 ? 1 : 2), 1);

  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  auto wait = [&](uint32_t b_, uint32_t par_) { return mbar_wait_sel<INLINE_WAIT>(b_, par_, abort_flag, kWaitBudgetNs); };
  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i) {
      const bool wide = (i >= QT_FULL && i < QT_FULL + 2) || (i >= P_FULL && i < P_FULL + 2) ||
                        (i >= X_FULL && i < X_FULL + 2) || (i >= L_FULL && i < L_FULL + 2);
      mbar_init(bar(i), wide ? kSlotThreads : 1);
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == kWarpMma) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  if (warp == kWarpLoad && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  pdl_trigger();
  pdl_wait();  // everything above touched only this CTA's shared and tensor memory
  DF_PTRACE(warp == kWarpMma ? 0 : (warp == 0 ? 1 : 2), 2);

  // Counting convention of every role: k = items of this CTA done so far, pos = K/V tiles of all
  // its items so far (ring stage pos & 1, phase (pos >> 1) & 1), stp = softmax steps of a slot so far.
  if (warp == kWarpLoad) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      Item it;
      uint32_t pos = 0, k = 0;
      bool ok = true;
      for (int r = 0; ok && item_of_round(p, &tab, r, &it); ++r, ++k) {
        for (int t = 0; t < 2; ++t) {
          // The landing buffer of slot t is free once the previous Q tile has been copied to tensor
          // memory and the O tile staged there before that has been read by its store.
          if (k >= 1 && !wait(bar(QT_FULL + t), (k - 1) & 1)) { ok = false; break; }
          if (k >= 2 && !wait(bar(LAND_FREE + t), (k - 2) & 1)) { ok = false; break; }
          mbar_arrive_expect_tx(bar(QL_FULL + t), kTile);
          // rows beyond the sequence are zero-filled by the copy engine
          tma_load_4d(aL + t * kTile, &tmQ, bar(QL_FULL + t), 0, (int)it.h, (int)(it.q0 + t * BM), (int)it.b);
          tma_load_4d(aL + t * kTile + kSlab, &tmQ, bar(QL_FULL + t), 32, (int)it.h, (int)(it.q0 + t * BM), (int)it.b);
        }
        for (int j = 0; ok && j < it.n_max; ++j, ++pos) {
          const uint32_t s = pos & 1, use = pos >> 1;
          if (use > 0 && !wait(bar(K_EMPTY + s), (use - 1) & 1)) { ok = false; break; }
          mbar_arrive_expect_tx(bar(K_FULL + s), kTile);
          tma_load_4d(aK + s * kTile, &tmK, bar(K_FULL + s), 0, (int)it.h, j * BN, (int)it.b);
          tma_load_4d(aK + s * kTile + kSlab, &tmK, bar(K_FULL + s), 32, (int)it.h, j * BN, (int)it.b);
          if (use > 0 && !wait(bar(V_EMPTY + s), (use - 1) & 1)) { ok = false; break; }
          mbar_arrive_expect_tx(bar(V_FULL + s), kTile);
          tma_load_4d(aV + s * kTile, &tmV, bar(V_FULL + s), 0, (int)it.h, j * BN, (int)it.b);
          tma_load_4d(aV + s * kTile + kSlab, &tmV, bar(V_FULL + s), 32, (int)it.h, j * BN, (int)it.b);
        }
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------ MMA issuer
    // Per item and key tile j: PV_A(j) QK_A(j+1) PV_B(j) QK_B(j+1). A slot that has issued its
    // last PV of the item goes straight on to the first QK of the next item (its Q is already in
    // tensor memory, the key tile already in the ring). Tile B never sees fewer key tiles than
    // tile A, so A is the first and B the last user of every K/V slot: A's products wait for the
    // slot, B's release it.
    // The whole warp runs this role, warp-uniformly; one elected lane issues the MMA and commit instructions and
    // every wait returns the same answer in all lanes (see elect_one).
    {
      auto wait = [&](uint32_t b_, uint32_t par_) {
        return __all_sync(0xffffffffu, mbar_wait_sel<INLINE_WAIT>(b_, par_, abort_flag, kWaitBudgetNs)) != 0;
      };
      const uint32_t idesc_qk = make_idesc(kFmtTF32, BM, BN, 0, 0);
      const uint32_t idesc_pv = make_idesc(kFmtTF32, BM, HD, 0, 1);
      // Descriptor low words of every K-step of both ring stages, computed once: inside a batch the warp then issues
      // nothing but MMAs (see mma_tf32_ts_lohi).
      const uint64_t dK0 = make_smem_desc(aK, 16, 1024, kSwz128), dV0 = make_smem_desc(aV, kSlab, 512, kSwz128B32);
      const uint32_t hiK = (uint32_t)(dK0 >> 32), hiV = (uint32_t)(dV0 >> 32);
      uint32_t loK[2][HD / 8], loV[2][BN / 8];
#pragma unroll
      for (int st = 0; st < 2; ++st) {
#pragma unroll
        for (int kk = 0; kk < HD / 8; ++kk)
          loK[st][kk] = (uint32_t)dK0 + ((st * kTile + (kk >> 2) * kSlab + (kk & 3) * 32) >> 4);
#pragma unroll
        for (int kk = 0; kk < BN / 8; ++kk) loV[st][kk] = (uint32_t)dV0 + ((st * kTile + kk * 1024) >> 4);
      }
      long long k_seen = -1, v_seen = -1;   // highest ring position whose K / V copy this thread has waited for
      uint32_t stp[2] = {0, 0};
      bool ok = true;
      // S_t = Q_t K^T for the key tile at ring position `pos`
      auto issue_qk = [&](int t, long long pos) -> bool {
        const int s = (int)(pos & 1);
        DF_PTRACE(0, 10 + t);
        if (pos > k_seen) {
          if (!wait(bar(K_FULL + s), (uint32_t)(pos >> 1) & 1)) return false;
          k_seen = pos;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + t * 128, a_tmem = tmem + 384 + t * HD;
        if (elect_one()) {
          if (s) {
            mma_tf32_ts_lohi(d_tmem, a_tmem, loK[1][0], hiK, idesc_qk, 0);
#pragma unroll
            for (int kk = 1; kk < HD / 8; ++kk) mma_tf32_ts_lohi_acc(d_tmem, a_tmem + kk * 8, loK[1][kk], hiK, idesc_qk);
          } else {
            mma_tf32_ts_lohi(d_tmem, a_tmem, loK[0][0], hiK, idesc_qk, 0);
#pragma unroll
            for (int kk = 1; kk < HD / 8; ++kk) mma_tf32_ts_lohi_acc(d_tmem, a_tmem + kk * 8, loK[0][kk], hiK, idesc_qk);
          }
          mma_commit(bar(S_FULL + t));
          if (t == 1) mma_commit(bar(K_EMPTY + s));
        }
        __syncwarp();
        DF_PTRACE(0, 12 + t);
        return true;
      };
      // O_t += P_t V for the key tile at ring position `pos`; `first` = first key tile of the item
      auto issue_pv = [&](int t, long long pos, bool first) -> bool {
        const int s = (int)(pos & 1);
        if (pos > v_seen) {
          if (!wait(bar(V_FULL + s), (uint32_t)(pos >> 1) & 1)) return false;
          v_seen = pos;
        }
        DF_PTRACE(0, 14 + t);
        if (!wait(bar(P_FULL + t), stp[t] & 1)) return false;
        DF_PTRACE(0, 16 + t);
        ++stp[t];
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + 256 + t * HD, a_tmem = tmem + t * 128;
        if (elect_one()) {
          if (s) {
            mma_tf32_ts_lohi(d_tmem, a_tmem, loV[1][0], hiV, idesc_pv, first ? 0u : 1u);
#pragma unroll
            for (int kk = 1; kk < BN / 8; ++kk) mma_tf32_ts_lohi_acc(d_tmem, a_tmem + kk * 8, loV[1][kk], hiV, idesc_pv);
          } else {
            mma_tf32_ts_lohi(d_tmem, a_tmem, loV[0][0], hiV, idesc_pv, first ? 0u : 1u);
#pragma unroll
            for (int kk = 1; kk < BN / 8; ++kk) mma_tf32_ts_lohi_acc(d_tmem, a_tmem + kk * 8, loV[0][kk], hiV, idesc_pv);
          }
          mma_commit(bar(O_FULL + t));
          if (t == 1) mma_commit(bar(V_EMPTY + s));
        }
        __syncwarp();
        DF_PTRACE(0, 18 + t);
        return true;
      };
      Item cur, nxt;
      int r = 0;
      uint32_t k = 0;
      long long base = 0;
      ok = item_of_round(p, &tab, 0, &cur);
      for (int t = 0; ok && t < 2; ++t) {
        ok = wait(bar(QT_FULL + t), 0);
        if (ok) ok = issue_qk(t, 0);
      }
      while (ok) {
        const bool has_nxt = item_of_round(p, &tab, r + 1, &nxt);
        for (int j = 0; ok && j < cur.n_max; ++j) {
          for (int t = 0; ok && t < 2; ++t) {
            if (j >= cur.n_kv[t]) continue;
            ok = issue_pv(t, base + j, j == 0);
            if (!ok) break;
            if (j + 1 < cur.n_kv[t]) {
              ok = issue_qk(t, base + j + 1);  // overwrites P_t(j) after PV_t(j) has read it
            } else if (has_nxt) {
              DF_PTRACE(0, 30 + t);
              ok = wait(bar(QT_FULL + t), (k + 1) & 1);
              if (ok) ok = issue_qk(t, base + cur.n_max);
            }
          }
        }
        if (!has_nxt) break;
        base += cur.n_max;
        cur = nxt;
        ++r;
        ++k;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue
    // The first kSlotWarps warps serve slot A, the next kSlotWarps slot B (a warp reads TMEM lanes 32*(w%4)..+31).
    // HALVES == 2: two warpgroups share every query row, warps 0-3 of a slot own key columns 0-63 of the K/V tile,
    // warps 4-7 columns 64-127; the row maximum is combined with the partner thread through shared memory, after
    // which both take identical rescale decisions. HALVES == 1: a thread owns its whole row.
    constexpr int CW = BN / HALVES;   // key columns per thread and step
    constexpr int NC = CW / 32;       // 32-column chunks of those
    constexpr int OW = HD / HALVES;   // O / Q dims per thread
    const int t = warp / kSlotWarps;
    const int quarter = warp & 3, half = (warp / 4) % HALVES;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + t * 128, tO = tmem + 256 + t * HD, tQ = tmem + 384 + t * HD;
    const int col0 = half * CW;
    float *xch = sXch + t * 768;
    // this thread's row in the slot's landing / staging buffer: OW dims = OW / 32 slab rows of 128 bytes, the first of
    // them here; 16-byte chunk c of row r sits at c ^ (r % 8) (128-byte swizzle of the tensor maps)
    uint8_t *land = smem + t * kTile + half * kSlab + row * 128;
    // Q rows of the item that landed k-th: shared memory -> tensor memory (TF32 already)
    auto q_to_tmem = [&](uint32_t kq) -> bool {
      if (!wait(bar(QL_FULL + t), kq & 1)) return false;
#pragma unroll
      for (int sl = 0; sl < OW / 32; ++sl) {
        uint32_t rq[32];
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          const uint4 v = *reinterpret_cast<const uint4 *>(land + sl * kSlab + ((x ^ (row & 7)) << 4));
          rq[4 * x] = v.x; rq[4 * x + 1] = v.y; rq[4 * x + 2] = v.z; rq[4 * x + 3] = v.w;
        }
        tmem_st32(tQ + lane_base + half * 32 + sl * 32, rq);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(QT_FULL + t));
      return true;
    };
    Item cur, nxt;
    uint32_t k = 0, stp = 0;
    int r = 0;
    bool ok = item_of_round(p, &tab, 0, &cur);
    if (ok) ok = q_to_tmem(0);
    while (ok) {
      const bool has_nxt = item_of_round(p, &tab, r + 1, &nxt);
      const long long i = cur.q0 + t * BM + row;
      const int nkv = cur.n_kv[t];
      long long kmax_ll = p.causal ? i + 1 : (long long)p.S;
      if (kmax_ll > (long long)p.S) kmax_ll = p.S;
      const int kmax = (int)kmax_ll;  // keys [0, kmax) are visible to this row
      float m_run = -INFINITY, m_used = -INFINITY;
      float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
      for (int j = 0; j < nkv; ++j, ++stp) {
        DF_PTRACE(1 + t, 20);
        if (!wait(bar(S_FULL + t), stp & 1)) { ok = false; break; }
        DF_PTRACE(1 + t, 21);
        tc_fence_after_sync();
        const int key0 = j * BN + col0;
        const bool need_mask = key0 + CW > kmax;
        // single pass: the thread's scores stay in registers from the maximum to the exponentials
        uint32_t rs[NC][32];
#pragma unroll
        for (int c = 0; c < NC; ++c) tmem_ld32(tS + lane_base + col0 + c * 32, rs[c]);
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int x = 0; x < 32; ++x)
              if (!(key0 + c * 32 + x < kmax)) rs[c][x] = 0xff800000u;  // -inf: exponentiates to 0
        }
        float mx_part;
        {
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
              mx0 = fmaxf(mx0, __uint_as_float(rs[c][x]));
              mx1 = fmaxf(mx1, __uint_as_float(rs[c][x + 1]));
              mx2 = fmaxf(mx2, __uint_as_float(rs[c][x + 2]));
              mx3 = fmaxf(mx3, __uint_as_float(rs[c][x + 3]));
            }
          mx_part = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        }
        float mx = mx_part;
        if (HALVES == 2) {
          // exchange the half-row maxima (double-buffered by step parity)
          float *xmax = xch + (stp & 1) * 256;
          xmax[half * 128 + row] = mx_part;
          mbar_arrive(bar(X_FULL + t));
          DF_PTRACE(1 + t, 22);
          if (!wait(bar(X_FULL + t), stp & 1)) { ok = false; break; }
          DF_PTRACE(1 + t, 23);
          mx = fmaxf(mx_part, xmax[(half ^ 1) * 128 + row]);
        }
        m_run = fmaxf(m_run, mx * p.scale_log2);
        // lazy rescale, decided per warp so that the TMEM accesses stay warp-uniform; a partner
        // warp sees the same rows and the same maxima, hence takes the same decision
        const bool want = (m_run - m_used > kRescaleThreshold) || (m_used == -INFINITY && m_run > -INFINITY);
        if (__any_sync(0xffffffffu, want)) {
          const float alpha = (m_used == -INFINITY) ? 0.0f : ex2_approx(m_used - m_run);
          l0 *= alpha; l1 *= alpha; l2 *= alpha; l3 *= alpha;
          m_used = m_run;
          if (j > 0) {
            if (!wait(bar(O_FULL + t), (stp - 1) & 1)) { ok = false; break; }
            tc_fence_after_sync();
            // each thread rescales its OW of the 64 O columns, 16 at a time to stay within the register budget
#pragma unroll 1
            for (int c = 0; c < OW / 16; ++c) {
              uint32_t ro[16];
              asm volatile(
                  "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                  : "=r"(ro[0]), "=r"(ro[1]), "=r"(ro[2]), "=r"(ro[3]), "=r"(ro[4]), "=r"(ro[5]), "=r"(ro[6]), "=r"(ro[7]),
                    "=r"(ro[8]), "=r"(ro[9]), "=r"(ro[10]), "=r"(ro[11]), "=r"(ro[12]), "=r"(ro[13]), "=r"(ro[14]), "=r"(ro[15])
                  : "r"(tO + lane_base + half * 32 + c * 16)
                  : "memory");
              tmem_wait_ld();
#pragma unroll
              for (int x = 0; x < 16; ++x) ro[x] = __float_as_uint(__uint_as_float(ro[x]) * alpha);
              asm volatile(
                  "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                  ::"r"(tO + lane_base + half * 32 + c * 16), "r"(ro[0]), "r"(ro[1]), "r"(ro[2]), "r"(ro[3]), "r"(ro[4]), "r"(ro[5]),
                    "r"(ro[6]), "r"(ro[7]), "r"(ro[8]), "r"(ro[9]), "r"(ro[10]), "r"(ro[11]), "r"(ro[12]), "r"(ro[13]), "r"(ro[14]),
                    "r"(ro[15])
                  : "memory");
            }
          }
        }
        DF_PTRACE(1 + t, 24);
        const float neg_m = (m_used == -INFINITY) ? 0.0f : -m_used;
        // P = 2^(s*scale_log2 - m) written over S with half a TF32 ulp added (the MMA drops the low mantissa bits: round
        // to nearest); the row sum takes the unrounded values (every thread of the row loaded its scores before the
        // exchange barrier above, so overwriting is safe)
#pragma unroll
        for (int c = 0; c < NC; ++c) {
#pragma unroll
          for (int x = 0; x < 32; x += 4) {
            const float e0 = ex2_approx(fmaf(__uint_as_float(rs[c][x]), p.scale_log2, neg_m));
            const float e1 = ex2_approx(fmaf(__uint_as_float(rs[c][x + 1]), p.scale_log2, neg_m));
            const float e2 = ex2_approx(fmaf(__uint_as_float(rs[c][x + 2]), p.scale_log2, neg_m));
            const float e3 = ex2_approx(fmaf(__uint_as_float(rs[c][x + 3]), p.scale_log2, neg_m));
            rs[c][x] = tf32_rna_operand(e0); rs[c][x + 1] = tf32_rna_operand(e1);
            rs[c][x + 2] = tf32_rna_operand(e2); rs[c][x + 3] = tf32_rna_operand(e3);
            l0 += e0; l1 += e1; l2 += e2; l3 += e3;
          }
          tmem_st32(tS + lane_base + col0 + c * 32, rs[c]);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar(P_FULL + t));
        DF_PTRACE(1 + t, 26);
      }
      if (!ok) break;
      // The last QK^T of this item has been consumed: the next item's Q rows can move into tensor
      // memory now, which lets the MMA thread start on that item while this one is being stored.
      DF_PTRACE(1 + t, 40);
      if (has_nxt && !q_to_tmem(k + 1)) { ok = false; break; }
      DF_PTRACE(1 + t, 41);
      float l = (l0 + l1) + (l2 + l3);
      // L_FULL completes once per item when a thread owns its row (staging done), twice when two share it (row sums
      // combined, staging done)
      uint32_t l_phase = HALVES == 2 ? 0u : (k & 1u);
      if (HALVES == 2) {
        // combine the two half-row sums
        float *xl = xch + 512;
        xl[half * 128 + row] = l;
        mbar_arrive(bar(L_FULL + t));
        if (!wait(bar(L_FULL + t), 0)) { ok = false; break; }
        l += xl[(half ^ 1) * 128 + row];
        l_phase = 1u;
      }
      if (!wait(bar(O_FULL + t), (stp - 1) & 1)) { ok = false; break; }
      tc_fence_after_sync();
      {
        // normalise and stage this thread's OW output columns
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll 1
        for (int sl = 0; sl < OW / 32; ++sl) {
          uint32_t ro[32];
          tmem_ld32(tO + lane_base + half * 32 + sl * 32, ro);
          tmem_wait_ld();
#pragma unroll
          for (int x = 0; x < 8; ++x)
            *reinterpret_cast<float4 *>(land + sl * kSlab + ((x ^ (row & 7)) << 4)) =
                make_float4(__uint_as_float(ro[4 * x]) * inv, __uint_as_float(ro[4 * x + 1]) * inv,
                            __uint_as_float(ro[4 * x + 2]) * inv, __uint_as_float(ro[4 * x + 3]) * inv);
        }
        if (half == 0 && p.lse && i < (long long)p.S)
          p.lse[((size_t)cur.b * p.H + cur.h) * p.S + (size_t)i] =
              l > 0.0f ? (m_used + lg2_approx(l)) * 0.6931471805599453f : -INFINITY;
      }
      // all threads of the slot have staged their rows; one thread hands the tile to the copy engine, which drops rows
      // beyond the sequence, and releases the buffer for the Q tile after next once the store has read it
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(bar(L_FULL + t));
      if (warp % kSlotWarps == 0 && lane == 0) {
        if (!wait(bar(L_FULL + t), l_phase)) { ok = false; break; }
        const long long qt = cur.q0 + t * BM;
        if (qt < (long long)p.S) {
          tma_store_4d(&tmO, aL + t * kTile, 0, (int)cur.h, (int)qt, (int)cur.b);
          tma_store_4d(&tmO, aL + t * kTile + kSlab, 32, (int)cur.h, (int)qt, (int)cur.b);
          tma_store_commit();
          tma_store_wait_read_all();
        }
        mbar_arrive(bar(LAND_FREE + t));
      }
      DF_PTRACE(1 + t, 42);
      if (!has_nxt) break;
      cur = nxt;
      ++r;
      ++k;
    }
  }

  // ---------------------------------------------------------------- teardown (all roles)
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    // error path only: give outstanding copies and MMAs a bounded chance to land before the
    // shared and tensor memory of this CTA are released
    if (warp == kWarpMma) {
      commit_elected(bar(DRAIN));  // by the lane that issued the MMAs: the election is deterministic
      for (int n = 0; n < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++n) {
      }
    }
    if (warp == kWarpLoad && lane == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
    }
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, DEV_STATUS_WAIT_EXPIRED);
    __syncthreads();
  }
  if (warp == kWarpMma) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

bool tensor_forward_persistent_supported(const AttnParams &p) {
  // DF_OPT_FWD_PERSIST: 0 = never, 2 = whenever the shape allows, default 1 = for sequences up to 2048.
  // Measured on B200 (H=12, B*S = 8192 or B = 1; TFLOP/s, this kernel against the one-CTA-per-pair kernel):
  // S = 1024 282 / 247, 2048 378 / 340, 4096 397 / 432, 8192 451 / 474, 16384 538 / 562, 32768 493 / 594. Short
  // sequences gain from set-up paid once per SM and from tiles overlapping across items; long ones lose because CTAs
  // launched in heaviest-first order walk the same K/V tiles at the same time and share them through L2.
  const int mode = option(DF_OPT_FWD_PERSIST);
  if (mode == 0 || (mode == 1 && p.Sq > 2048)) return false;
  if (p.bf16 || p.D != HD || p.Sq != p.Sk || p.shift != 0 || p.Sq == 0 || p.B == 0) return false;
  if ((uint64_t)p.B * p.H * ((p.Sq + 2 * BM - 1) / (2 * BM)) > 0x7fffffffull) return false;
  return true;  // alignment and scale are checked by tensor_forward_supported, which the caller has passed
}

namespace {
struct DeviceInfo {
  std::once_flag once;
  int n_sm = 0;
  bool ok = false;
};
DeviceInfo g_dev[64];
}  // namespace

int tensor_forward_persistent(const AttnParams &p, cudaStream_t s) {
  int dev = 0;
  if (check_cuda(cudaGetDevice(&dev)) != DF_OK) return DF_ERR_CUDA;
  if (dev < 0 || dev >= 64) return DF_ERR_CUDA;
  DeviceInfo &di = g_dev[dev];
  std::call_once(di.once, [&]() {
    di.ok = cudaFuncSetAttribute(k_attn_fwd_persist_tf32_d64<true, DF_FWD_HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal) == cudaSuccess &&
            cudaFuncSetAttribute(k_attn_fwd_persist_tf32_d64<false, DF_FWD_HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal) == cudaSuccess &&
            cudaDeviceGetAttribute(&di.n_sm, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && di.n_sm > 0;
  });
  if (!di.ok) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  const int n_sm = di.n_sm;
  CUtensorMap tmQ, tmK, tmV, tmO;
  // V is an MN-major 32-bit operand: 32-byte-atom swizzle; O is typed FLOAT32 so the store moves the words unchanged
  if (!encode_head_tile_map(&tmQ, p.q, false, HD, p.B, p.H, p.Sq, BM, false) ||
      !encode_head_tile_map(&tmK, p.k, false, HD, p.B, p.H, p.Sk, BN, false) ||
      !encode_head_tile_map(&tmV, p.v, false, HD, p.B, p.H, p.Sk, BN, true) ||
      !encode_head_tile_map(&tmO, p.out, false, HD, p.B, p.H, p.Sq, BM, false, true)) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  PParams fp;
  fp.out = p.out;
  fp.lse = p.lse;
  fp.B = p.B; fp.H = p.H; fp.S = p.Sq;
  fp.scale_log2 = p.scale * 1.4426950408889634f;
  fp.causal = p.causal;
  fp.n_pairs = (int)((p.Sq + 2 * BM - 1) / (2 * BM));
  fp.n_items = fp.n_pairs * (int)(p.B * p.H);
  fp.status = device_status_ptr();
  const dim3 grid(fp.n_items < n_sm ? fp.n_items : n_sm);
  // explicit work lists where the snake order leaves a heavy tail; weight = key tiles of the pair's
  // later query tile plus 3/4 of a step for the change of pair
  static thread_local SchedTable tab;
  const SchedKey key{0, p.B * p.H, p.Sq, p.Sk, p.causal, 0, (int)grid.x};
  schedule_for(key, fp.n_items, [](const void *c, int i) -> uint32_t {
    Item it;
    decode_item(*static_cast<const PParams *>(c), i, &it);
    return 4u * (uint32_t)it.n_max + 3u;
  }, &fp, &tab);
  // measured on B200 (B*H = 96 / 12): S = 1024 0.0536 vs 0.0559 ms with the loop inline; S = 8192 0.2644 vs 0.2609, S = 16384
  // 1.001 vs 0.968 with one out-of-line copy
  const cudaError_t launch_err =
      p.Sq <= 2048 ? launch_kernel(k_attn_fwd_persist_tf32_d64<true, DF_FWD_HALVES>, grid, dim3(kThreadsOf(DF_FWD_HALVES)), kSmemTotal, s, option(DF_OPT_PDL) != 0, tmQ,
                                   tmK, tmV, tmO, tab, fp)
                   : launch_kernel(k_attn_fwd_persist_tf32_d64<false, DF_FWD_HALVES>, grid, dim3(kThreadsOf(DF_FWD_HALVES)), kSmemTotal, s, option(DF_OPT_PDL) != 0, tmQ,
                                   tmK, tmV, tmO, tab, fp);
  note_launch();
#ifdef DF_ATTN_TRACE
  if (getenv("DF_ATTN_TRACE_DUMP")) {
    static unsigned long long host[3 * 1024];
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(host, g_pfwd_trace, sizeof(host));
    for (int slot = 0; slot < 3; ++slot)
      for (int e = 0; e < 511; ++e)
        if (host[slot * 1024 + 2 * e + 1])
          printf("ptrace slot %d ev %llu t %llu\n", slot, host[slot * 1024 + 2 * e], host[slot * 1024 + 2 * e + 1] - host[1]);
  }
#endif
  return check_cuda(launch_err);
}

}  // namespace df
