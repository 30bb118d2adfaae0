// attn_bwd_sm100.cu — fused causal attention backward for B200 (sm_100a), fp32 API, TF32 MMA.
//
// Replaces the arithmetic of kernel_mha_bwd_all_heads
// (darkforest-cuda/kernels/attention_fused.cu:390-516) from saved logsumexp and delta:
//   P = exp(scale*QK^T - lse)   dP = dO V^T   dS = P o (dP - delta)
//   dV = P^T dO                 dK = scale * dS^T Q        dQ = scale * dS K
// with no S x S scratch, no atomics (bit-reproducible) and no memsets: two kernels (a whole-sequence call runs
// dQ first, which also forms delta, then dK/dV), each recomputing P tile by tile on the tensor cores.
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
// MMA issue: tcgen05 MMAs of one thread execute in issue order, which is what lets single shared-memory stages
// suffice. The dQ kernel has one MMA warp that interleaves the phases of consecutive tiles (.., S_{j+1}, dP_{j+1},
// dQ_j, ..: dP has two buffers in tensor memory and runs a step ahead of dQ); the dK/dV kernel has one MMA warp per
// product chain (dV_i, S_{i+2} and dK_i, dP_{i+1}: they share
// nothing) and a second S^T buffer in tensor memory, so the tensor pipe has work while the compute warps are busy.
// An MMA role is run by all 32 lanes of its warp, warp-uniformly, with elect.sync around the tensor instructions.
// Both kernels are persistent (at most one CTA per SM, a static heaviest-first list of tiles per
// CTA, run as one uninterrupted pipeline) and hand finished tiles to the copy engine through
// shared memory. Tiles that become free at different times land on barriers of their own (K and V in the dK/dV
// kernel, Q and dO/O in the dQ kernel), so that an item's last accumulating product never queues behind the wait for
// a tile of the next item that it does not need.
//
// Inputs are rounded to TF32 by the TFLOAT32 tensor maps (nearest even); P and dS are rounded
// with cvt.rna before they are written back to TMEM. Every wait is bounded (see mbar_wait).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "df_common.cuh"
#include "sm100_ptx.cuh"

namespace df {
namespace {

using namespace ptx;

constexpr int BT = 128;  // tile edge: keys per CTA / queries per step (and vice versa)
constexpr int HD = 64;
constexpr int kBwdThreads = 352;  // dQ kernel: warps 0-7 compute, 8-9 TMA producers, 10 MMA issuer
// column groups of the dK/dV kernel's compute warps (2: 8 compute warps, 4: 16). Measured on the B200 with the same
// inputs and bit-identical results: 16 warps (96 registers each, the MMA warp sharing its scheduler with four of
// them) are 13 % slower than 8 (S = 16384: 1.59 ms against 1.40 ms).
#ifndef DF_KV_NSUB
#define DF_KV_NSUB 2
#endif
constexpr int kKvThreads = (4 * DF_KV_NSUB + 4) * 32;
constexpr uint32_t kSlab = 128 * 128;
constexpr uint32_t kTile = 2 * kSlab;
constexpr uint32_t kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;

// Optional phase trace (build with -DDF_ATTN_TRACE): (event id, SM clock) pairs recorded by the
// MMA thread (slot 0) and lane 0 of compute warp 0 (slot 1) of CTA 0 of the dK/dV kernel; the
// launcher prints them when DF_ATTN_TRACE_DUMP is set. Compiled out by default.
#ifdef DF_ATTN_TRACE
__device__ unsigned long long g_bwd_trace[2 * 1024];
#define DF_BTRACE(slot, id)                                           \
  do {                                                                \
    if (trace_on && tr_n < 511) {                                     \
      g_bwd_trace[(slot)*1024 + 2 * tr_n] = (id);                     \
      g_bwd_trace[(slot)*1024 + 2 * tr_n + 1] = clock64();            \
      ++tr_n;                                                         \
    }                                                                 \
  } while (0)
#else
#define DF_BTRACE(slot, id) do { } while (0)
#endif

struct BwdParams {
  const float *lse;
  const float *delta;
  float *delta_out;  // dQ kernel with fused row sums: delta = rowsum(dO o O) is computed there and written here
  float *dq, *dk, *dv;
  uint32_t B, H, Sq, Sk;
  float scale, scale_log2;
  int causal;
  long long shift;
  unsigned int *status;
};

// MMA batches. The descriptor words of every K-step of a tile are computed once per kernel (TileK / TileMN); a batch
// is then issued by ONE elected lane as nothing but tcgen05.mma instructions (and the commits that follow it): the
// issuing warp shares its scheduler with busy compute warps, and every other instruction between two MMAs costs the
// tensor pipe time (see mma_tf32_ts_lohi). Shared memory ends below 256 KB, so the 14-bit address field never carries.
struct TileK {   // K-major 128 x 64 fp32 tile of two 128-byte slabs: 8 K-steps
  uint32_t lo[HD / 8], hi;
};
struct TileMN {  // MN-major [128 rows (K), 64 dims (N)] tile: 16 K-steps
  uint32_t lo[BT / 8], hi;
};
__device__ __forceinline__ TileK tile_k(uint32_t tile_smem) {
  TileK t;
  const uint64_t d = make_smem_desc(tile_smem, 16, 1024, kSwz128);
  t.hi = (uint32_t)(d >> 32);
#pragma unroll
  for (int kk = 0; kk < HD / 8; ++kk) t.lo[kk] = (uint32_t)d + (((kk >> 2) * kSlab + (kk & 3) * 32) >> 4);
  return t;
}
__device__ __forceinline__ TileMN tile_mn(uint32_t tile_smem) {
  TileMN t;
  const uint64_t d = make_smem_desc(tile_smem, kSlab, 512, kSwz128B32);
  t.hi = (uint32_t)(d >> 32);
#pragma unroll
  for (int kk = 0; kk < BT / 8; ++kk) t.lo[kk] = (uint32_t)d + ((kk * 1024) >> 4);
  return t;
}
// To be called by the elected lane only.
// 8 K-steps of a 128x128x64 SS MMA, both operands K-major tiles.
__device__ __forceinline__ void batch_ss_128x128(uint32_t d_tmem, const TileK &a, const TileK &b, uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < HD / 8; ++kk) mma_tf32_ss_lohi(d_tmem, a.lo[kk], a.hi, b.lo[kk], b.hi, idesc, kk > 0 ? 1u : 0u);
}
// 16 K-steps of a 128x64x128 TS MMA: A = 128 TMEM columns, B = MN-major tile.
__device__ __forceinline__ void batch_ts_128x64(uint32_t d_tmem, uint32_t a_tmem, const TileMN &b, uint32_t idesc, bool accumulate) {
  mma_tf32_ts_lohi(d_tmem, a_tmem, b.lo[0], b.hi, idesc, accumulate ? 1u : 0u);
#pragma unroll
  for (int kk = 1; kk < BT / 8; ++kk) mma_tf32_ts_lohi_acc(d_tmem, a_tmem + kk * 8, b.lo[kk], b.hi, idesc);
}
// The dQ kernel keeps the other form - all lanes call these, one lane is elected per MMA, the descriptor is base +
// constant: with pure-MMA batches it measured 1.5 % faster at S = 1024 but 4 % slower at S = 16384 (the dK/dV kernel
// gained 1-3 % at both).
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile_smem) { return make_smem_desc(tile_smem, 16, 1024, kSwz128); }
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t tile_smem) { return make_smem_desc(tile_smem, kSlab, 512, kSwz128B32); }
__device__ __forceinline__ void issue_ss_128x128(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < HD / 8; ++kk) {
    const uint64_t off = (uint64_t)(((kk >> 2) * kSlab + (kk & 3) * 32) >> 4);
    if (elect_one()) mma_tf32_ss(d_tmem, a_desc + off, b_desc + off, idesc, kk > 0);
  }
}
__device__ __forceinline__ void issue_ts_128x64(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < BT / 8; ++kk)
    if (elect_one()) mma_tf32_ts(d_tmem, a_tmem + kk * 8, b_desc + (uint64_t)((kk * 1024) >> 4), idesc, (accumulate || kk > 0) ? 1u : 0u);
}
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap *m, uint32_t bar, int h, int row0, int b) {
  mbar_arrive_expect_tx(bar, kTile);
  tma_load_4d(dst, m, bar, 0, h, row0, b);
  tma_load_4d(dst + kSlab, m, bar, 32, h, row0, b);
}

// =========================================================================================
// Work distribution shared by both kernels
// =========================================================================================
// Both kernels are persistent: the grid has at most one CTA per SM and every CTA walks a static
// list of work items (one 128-row tile of one head each). Items are numbered heaviest first
// ((batch, head) fastest), dealt to the CTAs in rounds, odd rounds in reverse CTA order, which
// balances the causal triangle as well as a greedy longest-first assignment. A CTA runs its items
// as ONE pipeline: barrier phases are counted over all steps of all items, so the copies and the
// first two MMAs of the next item are in flight while the last products of the current item
// finish and its result tile is stored.
__device__ __forceinline__ int item_of_round(int r, int n_items) {
  return (int)snake_item(r, (int)gridDim.x, (int)blockIdx.x, n_items);
}

// =========================================================================================
// dK / dV
// =========================================================================================
namespace kv {
enum Bar { K_FULL = 0, V_FULL, K_EMPTY, V_EMPTY, QK_FULL, GK_FULL, QM_FULL, GM_FULL, QM_EMPTY, GM_EMPTY,
           S_FULL0, S_FULL1, DP_FULL, P_FULL0, P_FULL1, DS_FULL, STAT_FULL, ACC_FULL, EPI_FULL, DRAIN, NUM };
constexpr uint32_t kStats = 6 * kTile;             // lse2[3][128], delta[3][128]
constexpr uint32_t kBars = kStats + 6 * 128 * 4;
constexpr uint32_t kSmemTotal = kBars + 256 + 1024;

// One work item: 128 keys of one head and the query tiles that can see them.
struct Item {
  uint32_t b, h;
  long long k0;       // first key row
  long long i_begin;  // first query tile
  int n_it;           // number of query tiles (<= 0: nobody sees these keys)
};
__device__ __forceinline__ Item decode(const BwdParams &p, int idx) {
  Item it;
  const uint32_t n_bh = p.B * p.H, bh = (uint32_t)idx % n_bh;
  it.b = bh / p.H;
  it.h = bh % p.H;
  it.k0 = (long long)((uint32_t)idx / n_bh) * BT;  // key tile 0 sees the most queries: heaviest first
  long long q_first = p.causal ? it.k0 - p.shift : 0;
  if (q_first < 0) q_first = 0;
  it.i_begin = q_first / BT;
  const long long n_qt = ((long long)p.Sq + BT - 1) / BT;
  it.n_it = (int)(n_qt - it.i_begin);
  return it;
}
// first round >= r whose item has work; -1 when this CTA's list is exhausted
__device__ __forceinline__ int next_round(const BwdParams &p, int r, int n_items, Item *out) {
  for (;; ++r) {
    const int idx = item_of_round(r, n_items);
    if (idx < 0) return -1;
    *out = decode(p, idx);
    if (out->n_it > 0) return r;
  }
}
}  // namespace kv

// NSUB = column groups of the compute warps: 4 * NSUB compute warps (warp w: TMEM lanes 32 * (w % 4).., query
// columns (w / 4) * 128 / NSUB ..), then two producer warps and two MMA warps. (Which warp number issues the MMAs
// makes no difference: with the MMA role on warp 0 instead of the last warp the kernel took the same time.)
template <int NSUB>
__global__ void __launch_bounds__((4 * NSUB + 4) * 32, 1)
k_attn_bwd_dkdv_tf32_d64(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const __grid_constant__ CUtensorMap tmQk, const __grid_constant__ CUtensorMap tmGk,
                         const __grid_constant__ CUtensorMap tmQm, const __grid_constant__ CUtensorMap tmGm,
                         const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                         const BwdParams p, const int n_items) {
  using namespace kv;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aK = smem_u32(smem), aV = aK + kTile, aQk = aK + 2 * kTile, aGk = aK + 3 * kTile,
                 aQm = aK + 4 * kTile, aGm = aK + 5 * kTile;
  float *sLse2 = reinterpret_cast<float *>(smem + kStats);   // [3][128]
  float *sDelta = sLse2 + 384;                               // [3][128]
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kBars);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kBars + 192);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + kBars + 196);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kCW = 4 * NSUB;        // compute warps
  constexpr int kArrivals = kCW * 32;  // every compute thread arrives (one arrival per warp measured the same)
  constexpr int CPT = BT / NSUB;       // query columns per compute thread
  constexpr int NCH = CPT / 32;        // 32-column chunks per compute thread
  constexpr int kWarpLoadK = kCW, kWarpLoadM = kCW + 1, kWarpMma = kCW + 2, kWarpMma2 = kCW + 3, kWarpCompute0 = 0;
  const size_t dm = (size_t)p.H * HD;
#ifdef DF_ATTN_TRACE
#ifdef DF_ATTN_TRACE_DQ
  const bool trace_on = false;
#else
  const bool trace_on = blockIdx.x == 0 && lane == 0 && (warp == kWarpMma || warp == kWarpCompute0);
#endif
  int tr_n = 0;
#endif
  DF_BTRACE(warp == kWarpMma ? 0 : 1, 1);

  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM; ++i)
      mbar_init(bar(i), (i == P_FULL0 || i == P_FULL1 || i == DS_FULL || i == STAT_FULL || i == EPI_FULL) ? kArrivals : ((i == ACC_FULL || i == DRAIN) ? 2 : 1));
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == kWarpMma) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  // S^T / P^T is double-buffered (steps alternate between the two): S^T of step g+2 is issued as soon as dV of step g
  // has been, two steps ahead of the compute warps, so they never wait for it
  const uint32_t tS0 = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 320, tS1 = tmem + 384;
  pdl_trigger();
  pdl_wait();  // everything above touched only this CTA's shared and tensor memory

  // Counters every role keeps for itself: g = steps (query tiles) done over all items, n = items
  // done. A barrier used once per step is in phase g & 1, one used once per item in phase n & 1.
  if (warp == kWarpLoadK) {
    // ---------------------------------------------- producer: K, V per item; K-major Q and dO tiles per step
    if (lane == 0) {
      Item cur;
      uint32_t g = 0, n = 0;
      for (int r = next_round(p, 0, n_items, &cur); r >= 0; r = next_round(p, r + 1, n_items, &cur), ++n) {
        bool ok = true;
        if (n > 0 && !mbar_wait(bar(K_EMPTY), (n - 1) & 1, abort_flag)) break;
        // K and V land on barriers of their own: the next item's first S^T needs only K, and V can be replaced only
        // after the item's last dP^T, a step later. On one barrier the S^T / dV warp stood waiting for V at the end of
        // every item, with the item's last dV (whose P^T was ready) queued behind that wait: 2 K cycles per item.
        mbar_arrive_expect_tx(bar(K_FULL), kTile);
        tma_load_4d(aK, &tmK, bar(K_FULL), 0, (int)cur.h, (int)cur.k0, (int)cur.b);
        tma_load_4d(aK + kSlab, &tmK, bar(K_FULL), 32, (int)cur.h, (int)cur.k0, (int)cur.b);
        for (int it = 0; it < cur.n_it; ++it, ++g) {
          const int q0 = (int)((cur.i_begin + it) * BT);
          // the K-major Q (dO) buffer is free once the S^T (dP^T) product that read it has completed: the
          // barrier that hands that product to the compute warps tells this thread too
          if (g > 0 && !mbar_wait(bar(S_FULL0 + ((g - 1) & 1)), ((g - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          load_tile(aQk, &tmQk, bar(QK_FULL), (int)cur.h, q0, (int)cur.b);
          if (it == 0) {  // V follows the item's first Q tile: that one, like K, does not have to wait for V's buffer
            if (n > 0 && !mbar_wait(bar(V_EMPTY), (n - 1) & 1, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(bar(V_FULL), kTile);
            tma_load_4d(aV, &tmV, bar(V_FULL), 0, (int)cur.h, (int)cur.k0, (int)cur.b);
            tma_load_4d(aV + kSlab, &tmV, bar(V_FULL), 32, (int)cur.h, (int)cur.k0, (int)cur.b);
          }
          if (g > 0 && !mbar_wait(bar(DP_FULL), (g - 1) & 1, abort_flag)) { ok = false; break; }
          load_tile(aGk, &tmGk, bar(GK_FULL), (int)cur.h, q0, (int)cur.b);
        }
        if (!ok) break;
      }
    }
  } else if (warp == kWarpLoadM) {
    // ---------------------------------------------- producer: MN-major dO and Q tiles per step, result stores per item
    if (lane == 0) {
      Item cur;
      uint32_t g = 0, n = 0;
      for (int r = next_round(p, 0, n_items, &cur); r >= 0; r = next_round(p, r + 1, n_items, &cur), ++n) {
        bool ok = true;
        for (int it = 0; it < cur.n_it; ++it, ++g) {
          const int q0 = (int)((cur.i_begin + it) * BT);
          // the MN-major dO (Q) buffer is released by a commit of its own right after dV (dK) of the step before:
          // waiting for the next S^T (dP^T) product instead delayed these loads and measured 1-3 % slower
          if (g > 0 && !mbar_wait(bar(GM_EMPTY), (g - 1) & 1, abort_flag)) { ok = false; break; }
          load_tile(aGm, &tmGm, bar(GM_FULL), (int)cur.h, q0, (int)cur.b);
          if (g > 0 && !mbar_wait(bar(QM_EMPTY), (g - 1) & 1, abort_flag)) { ok = false; break; }
          load_tile(aQm, &tmQm, bar(QM_FULL), (int)cur.h, q0, (int)cur.b);
        }
        // The compute warps stage the item's dV and dK tiles in these two buffers; this thread
        // hands them to the copy engine (key rows beyond Sk are dropped) and may refill the
        // buffers for the next item once the store has read them.
        if (!ok || !mbar_wait(bar(EPI_FULL), n & 1, abort_flag)) break;
        tma_store_4d(&tmDV, aGm, 0, (int)cur.h, (int)cur.k0, (int)cur.b);
        tma_store_4d(&tmDV, aGm + kSlab, 32, (int)cur.h, (int)cur.k0, (int)cur.b);
        tma_store_4d(&tmDK, aQm, 0, (int)cur.h, (int)cur.k0, (int)cur.b);
        tma_store_4d(&tmDK, aQm + kSlab, 32, (int)cur.h, (int)cur.k0, (int)cur.b);
        tma_store_commit();
        tma_store_wait_read_all();
      }
    }
  } else if (warp == kWarpMma || warp == kWarpMma2) {
    // ---------------------------------------------- MMA issuers
    // The step's four products form two chains that share neither tensor memory nor operand buffers nor barriers:
    //   warp kWarpMma :  .., dV_g (needs P_g), S_{g+2} (overwrites P^T_g after dV_g has read it), ..
    //   warp kWarpMma2:  .., dK_g (needs dS_g), dP_{g+1} (overwrites dS^T_g after dK_g has read it), ..
    // Each chain has its own warp: MMAs of one thread execute in issue order, which is all a chain needs, and while
    // one warp sits between two batches (poll, fence, the first MMA's start-up) the other's MMAs keep the tensor
    // pipe busy. Step g+1 may belong to the next item (new K and V), so the pipe never drains between items.
    // The whole warp runs its role; only the MMA and commit instructions are issued by one elected lane.
    const uint32_t idesc_ss = make_idesc(kFmtTF32, BT, BT, 0, 0);
    const uint32_t idesc_ts = make_idesc(kFmtTF32, BT, HD, 0, 1);
    if (warp == kWarpMma) {
      // ---- chain S / dV. S^T runs two steps ahead of dV: a cursor of its own walks the flat sequence of steps.
      const TileK dA = tile_k(aK), dB = tile_k(aQk);
      const TileMN dM = tile_mn(aGm);
      Item s_item;
      int s_r = next_round(p, 0, n_items, &s_item), s_it = 0;
      uint32_t gs = 0, ns = 0;  // flat index and item ordinal of the next S^T to issue
      // S^T of the cursor's step into buffer gs & 1; false when a wait gave up
      auto issue_next_s = [&]() -> bool {
        DF_BTRACE(0, 10);
        if (s_it == 0) {  // first step of an item: its K tile must have landed
          if (!mbar_wait_warp(bar(K_FULL), ns & 1, abort_flag)) return false;
        }
        if (!mbar_wait_warp(bar(QK_FULL), gs & 1, abort_flag)) return false;
        tc_fence_after_sync();
        DF_BTRACE(0, 11);
        if (elect_one()) {
          batch_ss_128x128((gs & 1) ? tS1 : tS0, dA, dB, idesc_ss);
          mma_commit(bar(S_FULL0 + (gs & 1)));
          if (s_it + 1 == s_item.n_it) mma_commit(bar(K_EMPTY));  // last S^T of its item: K may be replaced
        }
        __syncwarp();
        DF_BTRACE(0, 12);
        ++gs;
        if (++s_it >= s_item.n_it) {
          s_r = next_round(p, s_r + 1, n_items, &s_item);
          s_it = 0;
          ++ns;
        }
        return true;
      };
      Item cur, nxt;
      uint32_t g = 0;
      int r = next_round(p, 0, n_items, &cur);
      bool ok = r >= 0;
      if (ok) ok = issue_next_s();
      if (ok && s_r >= 0) ok = issue_next_s();
      while (ok) {
        const int rn = next_round(p, r + 1, n_items, &nxt);
        for (int it = 0; ok && it < cur.n_it; ++it, ++g) {
          const bool last = it + 1 == cur.n_it;
          DF_BTRACE(0, 30);
          const uint32_t b = g & 1, ph2 = (g >> 1) & 1;
          const uint32_t m = mbar_test3_warp(bar(P_FULL0 + b), ph2, bar(GM_FULL), b, bar(GM_FULL), b);
          if ((!(m & 1u) && !mbar_wait_warp(bar(P_FULL0 + b), ph2, abort_flag)) || (!(m & 2u) && !mbar_wait_warp(bar(GM_FULL), b, abort_flag))) {
            ok = false;
            break;
          }
          DF_BTRACE(0, 31);
          tc_fence_after_sync();
          if (elect_one()) {
            batch_ts_128x64(tDV, b ? tS1 : tS0, dM, idesc_ts, it > 0);  // dV += P^T dO
            mma_commit(bar(GM_EMPTY));
            if (last) mma_commit(bar(ACC_FULL));  // the second of its two arrivals completes the item's accumulators
          }
          __syncwarp();
          DF_BTRACE(0, 32);
          // S^T of step g+2 goes into the buffer dV_g has just been issued on (MMAs of one thread run in order)
          if (s_r >= 0 && !issue_next_s()) { ok = false; break; }
        }
        if (rn < 0) break;
        r = rn;
        cur = nxt;
      }
    } else {
      // ---- chain dP / dK
      const TileK dA = tile_k(aV), dB = tile_k(aGk);
      const TileMN dM = tile_mn(aQm);
      Item cur, nxt;
      uint32_t g = 0, n = 0;
      int r = next_round(p, 0, n_items, &cur);
      bool ok = r >= 0;
      // dP^T of step gs; `last` = last step of its item: V may then be replaced;
      // `landed`: the caller has already seen the operand tile's barrier complete (and fenced after that)
      auto issue_dp = [&](uint32_t gs, bool last, bool landed) -> bool {
        if (!landed) {
          if (!mbar_wait_warp(bar(GK_FULL), gs & 1, abort_flag)) return false;
          tc_fence_after_sync();
        }
        if (elect_one()) {
          batch_ss_128x128(tDP, dA, dB, idesc_ss);
          mma_commit(bar(DP_FULL));
          if (last) mma_commit(bar(V_EMPTY));
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = mbar_wait_warp(bar(V_FULL), 0, abort_flag);
      if (ok) ok = issue_dp(0, cur.n_it == 1, false);
      while (ok) {
        const int rn = next_round(p, r + 1, n_items, &nxt);
        for (int it = 0; ok && it < cur.n_it; ++it, ++g) {
          const bool last = it + 1 == cur.n_it;
          const bool has_next = !last || rn >= 0;
          const bool next_last = last ? (nxt.n_it == 1) : (it + 2 == cur.n_it);
          // One poll covers what dK_g needs and the operand tile of the product issued right after it; only a
          // barrier that is still open is then waited for on its own.
          const uint32_t ph = g & 1, phn = ph ^ 1;
          const uint32_t m = mbar_test3_warp(bar(DS_FULL), ph, bar(QM_FULL), ph, bar(has_next ? GK_FULL : QM_FULL), has_next ? phn : ph);
          if ((!(m & 1u) && !mbar_wait_warp(bar(DS_FULL), ph, abort_flag)) || (!(m & 2u) && !mbar_wait_warp(bar(QM_FULL), ph, abort_flag))) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (elect_one()) {
            batch_ts_128x64(tDK, tDP, dM, idesc_ts, it > 0);  // dK += dS^T Q
            mma_commit(bar(QM_EMPTY));
            if (last) mma_commit(bar(ACC_FULL));
          }
          __syncwarp();
          if (has_next) {
            if (last) {
              if (!mbar_wait_warp(bar(V_FULL), (n + 1) & 1, abort_flag)) { ok = false; break; }
              tc_fence_after_sync();
            }
            if (!issue_dp(g + 1, next_last, (m & 4u) != 0u)) { ok = false; break; }  // overwrites dS^T_g after dK_g has read it
          }
        }
        if (rn < 0) break;
        r = rn;
        cur = nxt;
        ++n;
      }
    }
  } else {
    // ---------------------------------------------- compute warps: lanes = keys, columns = queries
    const int quarter = warp & 3, sub = (warp - kWarpCompute0) >> 2;
    const int row = quarter * 32 + lane;
    const int tid = threadIdx.x - kWarpCompute0 * 32;  // 0 .. 128 * NSUB - 1
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int col0 = sub * CPT;
    // result tiles: the first half of the column groups hands over dV, the second half scale * dK, each thread
    // kOutCols dims of its key row starting at out0
    constexpr int kOutCols = HD / (NSUB / 2);
    const bool is_dk = sub >= NSUB / 2;
    const int out0 = (sub % (NSUB / 2)) * kOutCols;
    // keys that no query sees: dK = dV = 0 (only with a causal shift or more keys than queries)
    for (int r0 = 0;; ++r0) {
      const int idx = item_of_round(r0, n_items);
      if (idx < 0) break;
      const Item z = decode(p, idx);
      if (z.n_it > 0) continue;
      const long long kj = z.k0 + row;
      if (kj < (long long)p.Sk) {
        float4 *dst = reinterpret_cast<float4 *>((is_dk ? p.dk : p.dv) + ((size_t)z.b * p.Sk + (size_t)kj) * dm + z.h * HD + out0);
#pragma unroll
        for (int x = 0; x < kOutCols / 4; ++x) dst[x] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    // row statistics of a query tile: threads 0-127 fetch lse, 128-255 fetch delta (the others none)
    // The value comes back RAW: nothing is computed from it here, so the thread does not stall on the load; it is
    // turned into what the phases use (`staged`) only when it is written to shared memory, a P phase later.
    auto fetch_stat = [&](const Item &im, int it) -> float {
      const long long q = (im.i_begin + it) * BT + (tid & 127);
      if (q >= (long long)p.Sq || tid >= 256) return (tid < 128) ? -INFINITY : 0.0f;
      const size_t s_base = ((size_t)im.b * p.H + im.h) * p.Sq;
      return __ldg((tid < 128 ? p.lse : p.delta) + s_base + q);
    };
    // lse in log2 units, +inf for a row without visible keys (P = 0); delta as it is
    auto staged = [&](float raw) -> float {
      if (tid >= 128) return raw;
      return (raw == -INFINITY) ? INFINITY : raw * kLog2e;
    };
    // Hands the finished accumulators of the CTA's item number `nd` to the second producer thread: half of the column
    // groups hand over dV, the other half scale * dK. Every MMA of the item has finished by then, so
    // the MN-major dO buffer stages dV and the MN-major Q buffer dK, in the 128-byte-swizzled
    // slab layout of the store's tensor map (16-byte chunk c of row r at c ^ (r % 8)).
    auto hand_over = [&](uint32_t nd) -> bool {
      if (!mbar_wait(bar(ACC_FULL), nd & 1, abort_flag)) return false;
      DF_BTRACE(1, 60);
      tc_fence_after_sync();
      const float mul = is_dk ? p.scale : 1.0f;
      uint8_t *stage = smem + (is_dk ? 4 : 5) * kTile + row * 128;
#pragma unroll 1
      for (int c = out0 / 32; c < (out0 + kOutCols) / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32((is_dk ? tDK : tDV) + lane_base + c * 32, rr);
        tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 8; ++x)
          *reinterpret_cast<float4 *>(stage + c * kSlab + ((x ^ (row & 7)) << 4)) =
              make_float4(__uint_as_float(rr[4 * x]) * mul, __uint_as_float(rr[4 * x + 1]) * mul,
                          __uint_as_float(rr[4 * x + 2]) * mul, __uint_as_float(rr[4 * x + 3]) * mul);
      }
      tc_fence_before_sync();  // the next item's first dV/dK overwrite the accumulators just read
      fence_proxy_async_smem();
      mbar_arrive(bar(EPI_FULL));
      DF_BTRACE(1, 61);
      return true;
    };
    Item cur, nxt;
    uint32_t g = 0, n = 0, gb = 0;  // gb = g % 3: the statistics buffer of step g
    int r = next_round(p, 0, n_items, &cur);
    bool ok = true;
    // Row statistics of a step are staged in shared memory ONE STEP AHEAD, in one of three buffers, and published
    // with a split barrier: every thread arrives in the middle of step g-1 (after its P phase) and waits at the
    // start of step g, by which time the slowest thread has long arrived. A thread that has passed the wait of step
    // g knows that all others are at least in step g-1, whose readers use buffers (g-1) % 3 and g % 3: writing buffer
    // (g+1) % 3 in step g is safe. (A barrier every step, with arrival and wait back to back, cost a quarter of the
    // compute warps' time: they all stood waiting for the slowest of them.)
    if (r >= 0) {
      const float s0 = staged(fetch_stat(cur, 0));
      if (tid < 128) sLse2[tid] = s0; else if (tid < 256) sDelta[tid - 128] = s0;
      mbar_arrive(bar(STAT_FULL));
    }
    while (r >= 0 && ok) {
      const int rn = next_round(p, r + 1, n_items, &nxt);
      for (int it = 0; it < cur.n_it; ++it, ++g) {
        const uint32_t ph = g & 1;
        const long long q0 = (cur.i_begin + it) * BT;
        const long long kj = cur.k0 + row;
        const float *lse2 = sLse2 + gb * 128, *dlt = sDelta + gb * 128;
        const uint32_t gb_next = gb == 2 ? 0 : gb + 1;
        // next step's statistics: loaded now, staged after the P phase below
        const bool has_next_step = it + 1 < cur.n_it || rn >= 0;
        float stat_next = 0.0f;
        if (it + 1 < cur.n_it) stat_next = fetch_stat(cur, it + 1);
        else if (rn >= 0) stat_next = fetch_stat(nxt, 0);
        if (!mbar_wait(bar(STAT_FULL), ph, abort_flag)) { ok = false; break; }
        // visible iff key <= query + shift  <=>  column >= kj - shift - q0
        const bool need_mask = p.causal && (q0 + p.shift < cur.k0 + (BT - 1));
        long long cmin_ll = kj - p.shift - q0;
        const int cmin = !need_mask ? 0 : (cmin_ll > BT ? BT : (cmin_ll < 0 ? 0 : (int)cmin_ll));
        DF_BTRACE(1, 50);
        const uint32_t tS = ph ? tS1 : tS0;
        if (!mbar_wait(bar(S_FULL0 + ph), (g >> 1) & 1, abort_flag)) { ok = false; break; }
        DF_BTRACE(1, 51);
        tc_fence_after_sync();
        float pr[CPT];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint32_t rr[32];
          tmem_ld32(tS + lane_base + col0 + c * 32, rr);
          tmem_wait_ld();
          // only a tile on the diagonal has hidden scores: they become -inf here (and 0 below), so that the
          // exponentials of every other tile carry no compare and select
          if (need_mask) {
#pragma unroll
            for (int x = 0; x < 32; ++x)
              if (col0 + c * 32 + x < cmin) rr[x] = 0xff800000u;
          }
          // the column statistics are the same for every lane: 128-bit broadcast reads
#pragma unroll
          for (int x4 = 0; x4 < 32; x4 += 4) {
            const float4 l4 = *reinterpret_cast<const float4 *>(lse2 + col0 + c * 32 + x4);
            const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int x = x4 + u;
              // rounded with the low bits cleared, so that one register serves as the P^T operand of dV and as P for dS
              // (keeping the unrounded value as well measured slower: 64 more live registers)
              rr[x] = cvt_rna_tf32(ex2_approx(fmaf(__uint_as_float(rr[x]), p.scale_log2, -lv[u])));
              pr[c * 32 + x] = __uint_as_float(rr[x]);
            }
          }
          tmem_st32(tS + lane_base + col0 + c * 32, rr);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar(P_FULL0 + ph));
        if (has_next_step) {
          const float sn = staged(stat_next);
          if (tid < 128) sLse2[gb_next * 128 + tid] = sn; else if (tid < 256) sDelta[gb_next * 128 + tid - 128] = sn;
          mbar_arrive(bar(STAT_FULL));
        }
        gb = gb_next;
        DF_BTRACE(1, 52);
        if (!mbar_wait(bar(DP_FULL), ph, abort_flag)) { ok = false; break; }
        DF_BTRACE(1, 53);
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint32_t rr[32];
          tmem_ld32(tDP + lane_base + col0 + c * 32, rr);
          tmem_wait_ld();
#pragma unroll
          for (int x4 = 0; x4 < 32; x4 += 4) {
            const float4 d4 = *reinterpret_cast<const float4 *>(dlt + col0 + c * 32 + x4);
            const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int x = x4 + u;
              rr[x] = tf32_rna_operand(pr[c * 32 + x] * (__uint_as_float(rr[x]) - dv[u]));
            }
          }
          tmem_st32(tDP + lane_base + col0 + c * 32, rr);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar(DS_FULL));
        DF_BTRACE(1, 54);
      }
      if (!ok || !hand_over(n)) { ok = false; break; }
      r = rn;
      cur = nxt;
      ++n;
    }
  }

  // ---------------------------------------------------------------- teardown (all roles)
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (warp == kWarpMma || warp == kWarpMma2) {
      commit_elected(bar(DRAIN));  // by the lane that issued the MMAs: the election is deterministic; two arrivals
      for (int t = 0; t < (1 << 16) && !mbar_try_wait(bar(DRAIN), 0); ++t) {
      }
    }
    if ((warp == kWarpLoadK || warp == kWarpLoadM) && lane == 0) {
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

// =========================================================================================
// dQ
// =========================================================================================
namespace dq {
enum Bar { Q_FULL = 0, GO_FULL, Q_EMPTY, G_EMPTY, KK_FULL, VK_FULL, KM_FULL, KM_EMPTY, S_FULL, S_FREE, DP_FULL0, DP_FULL1,
           DS_FULL, ACC_FULL, EPI_FULL, O_FREE, DX_FULL, DRAIN, NUM };
constexpr uint32_t kBars = 6 * kTile;              // Q, dO, K (K-major), V, K (MN-major), O (only with fused row sums)
constexpr uint32_t kXch = kBars + 256;             // partial row sums [2][128]
constexpr uint32_t kSmemTotal = kXch + 1024 + 1024;

// One work item: 128 queries of one head and the key tiles they can see.
struct Item {
  uint32_t b, h;
  long long q0;  // first query row
  int n_kv;      // number of key tiles (0: the rows see no key)
};
__device__ __forceinline__ Item decode(const BwdParams &p, int idx, int n_qt) {
  Item it;
  const uint32_t n_bh = p.B * p.H, bh = (uint32_t)idx % n_bh;
  it.b = bh / p.H;
  it.h = bh % p.H;
  it.q0 = (long long)(n_qt - 1 - (int)((uint32_t)idx / n_bh)) * BT;  // the latest query tile sees the most keys
  long long kv_end = p.causal ? it.q0 + (BT - 1) + p.shift + 1 : (long long)p.Sk;
  if (kv_end > (long long)p.Sk) kv_end = p.Sk;
  if (kv_end < 0) kv_end = 0;
  it.n_kv = (int)((kv_end + BT - 1) / BT);
  return it;
}
__device__ __forceinline__ int next_round(const BwdParams &p, int r, int n_items, int n_qt, Item *out) {
  for (;; ++r) {
    const int idx = item_of_round(r, n_items);
    if (idx < 0) return -1;
    *out = decode(p, idx, n_qt);
    if (out->n_kv > 0) return r;
  }
}
}  // namespace dq

// FUSE_DELTA: the kernel also fetches the O tile of its queries, computes delta = rowsum(dO o O)
// itself (dO as rounded to TF32 by its tensor map, the same values the dP product sees) and
// writes it to p.delta_out for the dK/dV kernel, which then has to run after this one.
template <bool FUSE_DELTA>
__global__ void __launch_bounds__(kBwdThreads, 1)
k_attn_bwd_dq_tf32_d64(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
                       const __grid_constant__ CUtensorMap tmKk, const __grid_constant__ CUtensorMap tmVk,
                       const __grid_constant__ CUtensorMap tmKm, const __grid_constant__ CUtensorMap tmDQ,
                       const __grid_constant__ CUtensorMap tmO, const BwdParams p, const int n_items) {
  using namespace dq;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aQ = smem_u32(smem), aG = aQ + kTile, aKk = aQ + 2 * kTile, aVk = aQ + 3 * kTile, aKm = aQ + 4 * kTile,
                 aO = aQ + 5 * kTile;
  float *sXch = reinterpret_cast<float *>(smem + kXch);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kBars);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kBars + 192);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(smem + kBars + 196);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t dm = (size_t)p.H * HD;
  const int n_qt = (int)(((long long)p.Sq + BT - 1) / BT);

  auto bar = [&](int id) { return smem_u32(&bars[id]); };
  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM; ++i) mbar_init(bar(i), (i == S_FREE || i == DS_FULL || i == EPI_FULL || i == O_FREE || i == DX_FULL) ? 256 : 1);
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
  // dP / dS is double-buffered (steps alternate): dP of step g+1 is issued ahead of dQ of step g, so the compute warps
  // never wait for it and the item's last dP - whose completion frees dO for the next item - runs a step early
  const uint32_t tS = tmem, tDP0 = tmem + 128, tDQ = tmem + 256, tDP1 = tmem + 320;
#ifdef DF_ATTN_TRACE
  // with -DDF_ATTN_TRACE_DQ the trace follows this kernel instead of the dK/dV kernel (same two slots)
#ifdef DF_ATTN_TRACE_DQ
  const bool trace_on = blockIdx.x == 0 && lane == 0 && (warp == 10 || warp == 0);
#else
  const bool trace_on = false;
#endif
  int tr_n = 0;
#endif
  pdl_trigger();
  pdl_wait();  // everything above touched only this CTA's shared and tensor memory

  // g = steps (key tiles) done over all items, n = items done (see the dK/dV kernel)
  if (warp == 8) {
    // ---------------------------------------------- producer: Q, dO per item; K-major K and V tiles per step
    if (lane == 0) {
      Item cur;
      uint32_t g = 0, n = 0;
      for (int r = next_round(p, 0, n_items, n_qt, &cur); r >= 0; r = next_round(p, r + 1, n_items, n_qt, &cur), ++n) {
        bool ok = true;
        if (n > 0 && !mbar_wait(bar(Q_EMPTY), (n - 1) & 1, abort_flag)) break;
        // Q lands on a barrier of its own, dO (and O) on another: the next item's first S needs only Q, whose buffer
        // is free a step before dO's. On one barrier the MMA warp stood waiting for all three tiles at the end of every
        // item with the item's last dQ queued behind that wait, and the compute warps behind it.
        mbar_arrive_expect_tx(bar(Q_FULL), kTile);
        tma_load_4d(aQ, &tmQ, bar(Q_FULL), 0, (int)cur.h, (int)cur.q0, (int)cur.b);
        tma_load_4d(aQ + kSlab, &tmQ, bar(Q_FULL), 32, (int)cur.h, (int)cur.q0, (int)cur.b);
        for (int j = 0; j < cur.n_kv; ++j, ++g) {
          // a K-major K (V) buffer is free once the S (dP) product that read it has completed
          if (g > 0 && !mbar_wait(bar(S_FULL), (g - 1) & 1, abort_flag)) { ok = false; break; }
          load_tile(aKk, &tmKk, bar(KK_FULL), (int)cur.h, j * BT, (int)cur.b);
          if (j == 0) {  // dO (and O) follow the item's first K tile, which does not have to wait for their buffers
            if (n > 0 && !mbar_wait(bar(G_EMPTY), (n - 1) & 1, abort_flag)) { ok = false; break; }
            // with fused row sums the compute warps read the dO and O tiles too: both are replaced
            // only after they are done with them
            if (FUSE_DELTA && n > 0 && !mbar_wait(bar(O_FREE), (n - 1) & 1, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(bar(GO_FULL), (FUSE_DELTA ? 2 : 1) * kTile);
            tma_load_4d(aG, &tmG, bar(GO_FULL), 0, (int)cur.h, (int)cur.q0, (int)cur.b);
            tma_load_4d(aG + kSlab, &tmG, bar(GO_FULL), 32, (int)cur.h, (int)cur.q0, (int)cur.b);
            if (FUSE_DELTA) {
              tma_load_4d(aO, &tmO, bar(GO_FULL), 0, (int)cur.h, (int)cur.q0, (int)cur.b);
              tma_load_4d(aO + kSlab, &tmO, bar(GO_FULL), 32, (int)cur.h, (int)cur.q0, (int)cur.b);
            }
          }
          if (g > 0 && !mbar_wait(bar(DP_FULL0 + ((g - 1) & 1)), ((g - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          load_tile(aVk, &tmVk, bar(VK_FULL), (int)cur.h, j * BT, (int)cur.b);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------- producer: MN-major K tiles per step, result store per item
    if (lane == 0) {
      Item cur;
      uint32_t g = 0, n = 0;
      for (int r = next_round(p, 0, n_items, n_qt, &cur); r >= 0; r = next_round(p, r + 1, n_items, n_qt, &cur), ++n) {
        bool ok = true;
        for (int j = 0; j < cur.n_kv; ++j, ++g) {
          // the buffer is released by a commit of its own right after dQ of the step before
          if (g > 0 && !mbar_wait(bar(KM_EMPTY), (g - 1) & 1, abort_flag)) { ok = false; break; }
          load_tile(aKm, &tmKm, bar(KM_FULL), (int)cur.h, j * BT, (int)cur.b);
        }
        // the compute warps stage the item's dQ tile in this buffer; hand it to the copy engine
        // (rows beyond Sq are dropped) and refill the buffer once the store has read it
        if (!ok || !mbar_wait(bar(EPI_FULL), n & 1, abort_flag)) break;
        tma_store_4d(&tmDQ, aKm, 0, (int)cur.h, (int)cur.q0, (int)cur.b);
        tma_store_4d(&tmDQ, aKm + kSlab, 32, (int)cur.h, (int)cur.q0, (int)cur.b);
        tma_store_commit();
        tma_store_wait_read_all();
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------- MMA issuer: .., S_{g+1}, dP_{g+1}, dQ_g, .. over all items
    // (at the last step of an item: S of the next item, dQ_g, then the next item's first dP)
    // (the whole warp runs this role; only the MMA and commit instructions are issued by one elected lane)
    {
      const uint32_t idesc_ss = make_idesc(kFmtTF32, BT, BT, 0, 0);
      const uint32_t idesc_ts = make_idesc(kFmtTF32, BT, HD, 0, 1);
      const uint64_t dQ_ = kmajor_desc(aQ), dG_ = kmajor_desc(aG), dKk = kmajor_desc(aKk), dVk = kmajor_desc(aVk), dKm = mnmajor_desc(aKm);
      Item cur, nxt;
      uint32_t g = 0, n = 0;
      int r = next_round(p, 0, n_items, n_qt, &cur);
      bool ok = r >= 0;
      // `last` = last step of its item: Q (for S) or dO (for dP) may then be replaced
      // `landed`: the caller has already seen the operand tile's barrier complete
      auto issue_s = [&](uint32_t gs, bool last, bool landed) -> bool {
        if (!landed) {
          if (!mbar_wait_warp(bar(KK_FULL), gs & 1, abort_flag)) return false;
          tc_fence_after_sync();
        }
        issue_ss_128x128(tS, dQ_, dKk, idesc_ss);  // S = Q K^T
        commit_elected(bar(S_FULL));
        if (last) commit_elected(bar(Q_EMPTY));
        return true;
      };
      auto issue_dp = [&](uint32_t gs, bool last) -> bool {
        if (!mbar_wait_warp(bar(VK_FULL), gs & 1, abort_flag)) return false;
        tc_fence_after_sync();
        issue_ss_128x128((gs & 1) ? tDP1 : tDP0, dG_, dVk, idesc_ss);  // dP = dO V^T
        commit_elected(bar(DP_FULL0 + (gs & 1)));
        if (last) commit_elected(bar(G_EMPTY));
        return true;
      };
      if (ok) ok = mbar_wait_warp(bar(Q_FULL), 0, abort_flag);
      if (ok) ok = issue_s(0, cur.n_kv == 1, false);
      if (ok) ok = mbar_wait_warp(bar(GO_FULL), 0, abort_flag);
      if (ok) ok = issue_dp(0, cur.n_kv == 1);
      while (ok) {
        const int rn = next_round(p, r + 1, n_items, n_qt, &nxt);
        for (int j = 0; ok && j < cur.n_kv; ++j, ++g) {
          const bool last = j + 1 == cur.n_kv;
          const bool has_next = !last || rn >= 0;
          const bool next_last = last ? (nxt.n_kv == 1) : (j + 2 == cur.n_kv);
          const uint32_t ph = g & 1, phn = ph ^ 1;
          if (has_next) {
            // S_{g+1} may overwrite S_g once the compute warps hold P_g in registers; one poll covers that and
            // the operand tile, only a barrier that is still open is then waited for on its own
            const uint32_t m = mbar_test3_warp(bar(S_FREE), ph, bar(KK_FULL), phn, bar(KK_FULL), phn);
            if (!(m & 1u) && !mbar_wait_warp(bar(S_FREE), ph, abort_flag)) { ok = false; break; }
            DF_BTRACE(0, 10);
            if (last && !mbar_wait_warp(bar(Q_FULL), (n + 1) & 1, abort_flag)) { ok = false; break; }
            DF_BTRACE(0, 11);
            tc_fence_after_sync();
            if (!issue_s(g + 1, next_last, (m & 2u) != 0u)) { ok = false; break; }
            DF_BTRACE(0, 12);
            // dP_{g+1} of the same item goes out now, into the buffer dQ_{g-1} (issued a step ago by this thread) read
            if (!last && !issue_dp(g + 1, next_last)) { ok = false; break; }
          }
          const uint32_t m = mbar_test3_warp(bar(DS_FULL), ph, bar(KM_FULL), ph, bar(KM_FULL), ph);
          if ((!(m & 1u) && !mbar_wait_warp(bar(DS_FULL), ph, abort_flag)) || (!(m & 2u) && !mbar_wait_warp(bar(KM_FULL), ph, abort_flag))) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          DF_BTRACE(0, 31);
          issue_ts_128x64(tDQ, ph ? tDP1 : tDP0, dKm, idesc_ts, j > 0);  // dQ += dS K
          DF_BTRACE(0, 32);
          commit_elected(bar(KM_EMPTY));
          if (last) commit_elected(bar(ACC_FULL));
          if (has_next && last) {
            // the first dP of the next item needs its dO tile, which can only be loaded once this item's last dP is
            // done: it follows the item's last dQ, so that the finished accumulator never waits behind that tile
            if (!mbar_wait_warp(bar(GO_FULL), (n + 1) & 1, abort_flag)) { ok = false; break; }
            if (!issue_dp(g + 1, next_last)) { ok = false; break; }
          }
          DF_BTRACE(0, 33);
        }
        if (rn < 0) break;
        r = rn;
        cur = nxt;
        ++n;
      }
    }
  } else {
    // ---------------------------------------------- compute warps: lanes = queries, columns = keys
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int col0 = half * 64;
    // query rows that see no key: dQ = 0
    for (int r0 = 0;; ++r0) {
      const int idx = item_of_round(r0, n_items);
      if (idx < 0) break;
      const Item z = decode(p, idx, n_qt);
      if (z.n_kv > 0) continue;
      const long long i = z.q0 + row;
      if (i < (long long)p.Sq) {
        float4 *dst = reinterpret_cast<float4 *>(p.dq + ((size_t)z.b * p.Sq + (size_t)i) * dm + z.h * HD + half * 32);
#pragma unroll
        for (int x = 0; x < 8; ++x) dst[x] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    // logsumexp (in log2 units) and delta of this thread's query row in item `im`
    // The logsumexp comes back RAW (-inf for a row beyond the sequence): nothing is computed from it here, so the
    // thread does not stall on the load; lse2_of() turns it into log2 units when the item starts.
    auto fetch_stats = [&](const Item &im, float *lse_raw, float *dlt) {
      const long long i = im.q0 + row;
      *lse_raw = -INFINITY;
      *dlt = 0.0f;
      if (i < (long long)p.Sq) {
        const size_t s_idx = ((size_t)im.b * p.H + im.h) * p.Sq + (size_t)i;
        *lse_raw = __ldg(p.lse + s_idx);
        if (!FUSE_DELTA) *dlt = __ldg(p.delta + s_idx);
      }
    };
    auto lse2_of = [](float raw) -> float { return (raw == -INFINITY) ? INFINITY : raw * kLog2e; };
    // Fused row sums: delta of this thread's row of item `im` (the nn-th item of this CTA) from the
    // dO and O tiles in shared memory. Each of the row's two threads sums its 32 dims (one
    // 128-byte slab row, 16-byte chunk c at c ^ (row % 8)); the halves meet in shared memory.
    auto fused_delta = [&](const Item &im, uint32_t nn, float *out) -> bool {
      if (!mbar_wait(bar(GO_FULL), nn & 1, abort_flag)) return false;
      const uint8_t *g_row = smem + kTile + half * kSlab + row * 128;
      const uint8_t *o_row = smem + 5 * kTile + half * kSlab + row * 128;
      float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        const uint32_t off = (uint32_t)((x ^ (row & 7)) << 4);
        const float4 gv = *reinterpret_cast<const float4 *>(g_row + off);
        const float4 ov = *reinterpret_cast<const float4 *>(o_row + off);
        acc0 = fmaf(gv.x, ov.x, acc0); acc1 = fmaf(gv.y, ov.y, acc1);
        acc0 = fmaf(gv.z, ov.z, acc0); acc1 = fmaf(gv.w, ov.w, acc1);
      }
      float *xs = sXch + (nn & 1) * 256;
      xs[half * 128 + row] = acc0 + acc1;
      mbar_arrive(bar(O_FREE));
      mbar_arrive(bar(DX_FULL));
      if (!mbar_wait(bar(DX_FULL), nn & 1, abort_flag)) return false;
      *out = xs[row] + xs[128 + row];
      const long long i = im.q0 + row;
      if (half == 0 && i < (long long)p.Sq) p.delta_out[((size_t)im.b * p.H + im.h) * p.Sq + (size_t)i] = *out;
      return true;
    };
    Item cur, nxt;
    uint32_t g = 0, n = 0;
    int r = next_round(p, 0, n_items, n_qt, &cur);
    bool ok = true;
    float lse_raw = -INFINITY, dlt = 0.0f, lse_raw_next = -INFINITY, dlt_next = 0.0f;
    if (r >= 0) fetch_stats(cur, &lse_raw, &dlt);
    if (FUSE_DELTA && r >= 0) ok = fused_delta(cur, 0, &dlt);
    while (r >= 0 && ok) {
      const int rn = next_round(p, r + 1, n_items, n_qt, &nxt);
      if (rn >= 0) fetch_stats(nxt, &lse_raw_next, &dlt_next);  // in flight while this item computes
      const float lse2 = lse2_of(lse_raw);
      const long long i = cur.q0 + row;
      long long kmax_ll = p.causal ? i + p.shift + 1 : (long long)p.Sk;
      if (kmax_ll > (long long)p.Sk) kmax_ll = p.Sk;
      if (kmax_ll < 0) kmax_ll = 0;
      const int kmax = (int)kmax_ll;
      for (int j = 0; j < cur.n_kv; ++j, ++g) {
        const uint32_t ph = g & 1;
        const int key0 = j * BT;
        const bool need_mask = key0 + BT > kmax;
        DF_BTRACE(1, 50);
        if (!mbar_wait(bar(S_FULL), ph, abort_flag)) { ok = false; break; }
        DF_BTRACE(1, 51);
        tc_fence_after_sync();
        float pr[64];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rr[32];
          tmem_ld32(tS + lane_base + col0 + c * 32, rr);
          tmem_wait_ld();
          // only the last key tiles of a row have hidden scores: they become -inf here (and 0 below), so that the
          // exponentials of every other tile carry no compare and select
          if (need_mask) {
#pragma unroll
            for (int x = 0; x < 32; ++x)
              if (!(key0 + col0 + c * 32 + x < kmax)) rr[x] = 0xff800000u;
          }
#pragma unroll
          for (int x = 0; x < 32; ++x) pr[c * 32 + x] = ex2_approx(fmaf(__uint_as_float(rr[x]), p.scale_log2, -lse2));
        }
        tc_fence_before_sync();
        mbar_arrive(bar(S_FREE));
        DF_BTRACE(1, 52);
        if (!mbar_wait(bar(DP_FULL0 + ph), (g >> 1) & 1, abort_flag)) { ok = false; break; }
        DF_BTRACE(1, 53);
        tc_fence_after_sync();
        const uint32_t tDP = ph ? tDP1 : tDP0;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rr[32];
          tmem_ld32(tDP + lane_base + col0 + c * 32, rr);
          tmem_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; ++x) rr[x] = tf32_rna_operand(pr[c * 32 + x] * (__uint_as_float(rr[x]) - dlt));
          tmem_st32(tDP + lane_base + col0 + c * 32, rr);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar(DS_FULL));
        DF_BTRACE(1, 54);
      }
      // the next item's dO and O tiles are on their way or already here: its row sums are
      // computed while the last dQ product of this item is still running (handing the finished dQ over first,
      // and the row sums after it, measured the same)
      if (FUSE_DELTA && ok && rn >= 0) ok = fused_delta(nxt, n + 1, &dlt_next);
      DF_BTRACE(1, 59);
      if (!ok || !mbar_wait(bar(ACC_FULL), n & 1, abort_flag)) { ok = false; break; }
      DF_BTRACE(1, 60);
      tc_fence_after_sync();
      {
        uint32_t rr[32];
        tmem_ld32(tDQ + lane_base + half * 32, rr);  // each half handles 32 of the 64 dims = one 128-byte slab
        tmem_wait_ld();
        // staged over the MN-major K buffer (free: every MMA of the item has finished) in the
        // swizzled slab layout of the store's tensor map; the second producer thread stores it
        uint8_t *stage = smem + 4 * kTile + half * kSlab + row * 128;
#pragma unroll
        for (int x = 0; x < 8; ++x)
          *reinterpret_cast<float4 *>(stage + ((x ^ (row & 7)) << 4)) =
              make_float4(__uint_as_float(rr[4 * x]) * p.scale, __uint_as_float(rr[4 * x + 1]) * p.scale,
                          __uint_as_float(rr[4 * x + 2]) * p.scale, __uint_as_float(rr[4 * x + 3]) * p.scale);
        tc_fence_before_sync();
        fence_proxy_async_smem();
        mbar_arrive(bar(EPI_FULL));
        DF_BTRACE(1, 61);
      }
      r = rn;
      cur = nxt;
      lse_raw = lse_raw_next;
      dlt = dlt_next;
      ++n;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (warp == 10) {
      commit_elected(bar(DRAIN));  // by the lane that issued the MMAs: the election is deterministic
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
  if (option(DF_OPT_DISABLE_TENSOR) != 0) return false;
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

namespace {
// Per device: kernel attributes and SM count, set up once under a lock.
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
    d.ok = cudaFuncSetAttribute(k_attn_bwd_dkdv_tf32_d64<DF_KV_NSUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kv::kSmemTotal) == cudaSuccess &&
           cudaFuncSetAttribute(k_attn_bwd_dq_tf32_d64<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dq::kSmemTotal) == cudaSuccess &&
           cudaFuncSetAttribute(k_attn_bwd_dq_tf32_d64<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dq::kSmemTotal) == cudaSuccess &&
           cudaDeviceGetAttribute(&d.n_sm, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && d.n_sm > 0;
  });
  if (!d.ok) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  *n_sm = d.n_sm;
  return DF_OK;
}

// Side stream of the block backward. The dQ and dK/dV kernels of a block call do not depend on
// each other; with one CTA per SM each, running them on two streams lets the CTAs of one start on
// SMs that the other has already left. The side stream and its fork/join events belong to the
// CALLING THREAD (one set per thread and device), so concurrent callers never record each
// other's events. They are created by df_attn_init or by the thread's first block backward on the
// device (the only place the library creates a CUDA object) and destroyed when the thread exits.
struct SideStreams {
  struct Side { cudaStream_t stream = nullptr; cudaEvent_t fork = nullptr, join = nullptr; bool ok = false, tried = false; };
  Side dev[64];
  ~SideStreams() {
    for (Side &sd : dev)
      if (sd.ok) {  // errors ignored: at process exit the driver may already be gone
        cudaEventDestroy(sd.fork);
        cudaEventDestroy(sd.join);
        cudaStreamDestroy(sd.stream);
      }
  }
  Side *get() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return nullptr;
    Side &sd = dev[d];
    if (!sd.tried) {
      sd.tried = true;
      sd.ok = cudaStreamCreateWithFlags(&sd.stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&sd.fork, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&sd.join, cudaEventDisableTiming) == cudaSuccess;
    }
    return sd.ok ? &sd : nullptr;
  }
};
thread_local SideStreams t_side;

// Events that df_attn_backward_profile asks the launcher to record around the two kernels.
thread_local cudaEvent_t *t_profile_events = nullptr;
}  // namespace

int tensor_backward_init() {
  int n_sm = 0;
  if (device_info(&n_sm) != DF_OK) return DF_ERR_CUDA;
  return t_side.get() ? DF_OK : DF_ERR_CUDA;
}

void tensor_backward_set_profile_events(cudaEvent_t *three_events) { t_profile_events = three_events; }

int tensor_backward(const AttnParams &p, cudaStream_t s) {
  int n_sm = 0;
  if (device_info(&n_sm) != DF_OK) return DF_ERR_CUDA;
  // Row sums fused into the dQ kernel when the caller passes O and a delta buffer to fill instead of
  // ready-made row sums; the dK/dV kernel then runs after the dQ kernel on the same stream.
  const bool fuse = p.delta_in == nullptr && p.o_in != nullptr && p.delta != nullptr;
  if (!fuse && p.delta_in == nullptr) return DF_ERR_INVALID_ARG;
  CUtensorMap tmQk, tmQm, tmGk, tmGm, tmKk, tmKm, tmVk, tmDQ, tmDK, tmDV, tmO;
  if (!encode_head_tile_map(&tmQk, p.q, false, HD, p.B, p.H, p.Sq, BT, false) ||
      !encode_head_tile_map(&tmQm, p.q, false, HD, p.B, p.H, p.Sq, BT, true) ||
      !encode_head_tile_map(&tmGk, p.d_out, false, HD, p.B, p.H, p.Sq, BT, false) ||
      !encode_head_tile_map(&tmGm, p.d_out, false, HD, p.B, p.H, p.Sq, BT, true) ||
      !encode_head_tile_map(&tmKk, p.k, false, HD, p.B, p.H, p.Sk, BT, false) ||
      !encode_head_tile_map(&tmKm, p.k, false, HD, p.B, p.H, p.Sk, BT, true) ||
      !encode_head_tile_map(&tmVk, p.v, false, HD, p.B, p.H, p.Sk, BT, false) ||
      !encode_head_tile_map(&tmDQ, p.d_q, false, HD, p.B, p.H, p.Sq, BT, false, true) ||
      !encode_head_tile_map(&tmDK, p.d_k, false, HD, p.B, p.H, p.Sk, BT, false, true) ||
      !encode_head_tile_map(&tmDV, p.d_v, false, HD, p.B, p.H, p.Sk, BT, false, true) ||
      !encode_head_tile_map(&tmO, fuse ? p.o_in : p.q, false, HD, p.B, p.H, p.Sq, BT, false, true)) {
    note_status(DF_ERR_CUDA);
    return DF_ERR_CUDA;
  }
  BwdParams bp;
  bp.lse = p.lse_in;
  bp.delta = fuse ? p.delta : p.delta_in;
  bp.delta_out = fuse ? p.delta : nullptr;
  bp.dq = p.d_q; bp.dk = p.d_k; bp.dv = p.d_v;
  bp.B = p.B; bp.H = p.H; bp.Sq = p.Sq; bp.Sk = p.Sk;
  bp.scale = p.scale;
  bp.scale_log2 = p.scale * kLog2e;
  bp.causal = p.causal;
  bp.shift = p.shift;
  bp.status = device_status_ptr();
  // persistent grids: one CTA per SM at most, each walking its share of the items
  const int items_kv = (int)(((p.Sk + BT - 1) / BT) * p.B * p.H);
  const int items_q = (int)(((p.Sq + BT - 1) / BT) * p.B * p.H);
  const dim3 grid_kv(items_kv < n_sm ? items_kv : n_sm);
  const dim3 grid_q(items_q < n_sm ? items_q : n_sm);
  cudaEvent_t *prof = t_profile_events;
  const bool pdl = option(DF_OPT_PDL) != 0 && prof == nullptr;
  SideStreams::Side *sd = (!fuse && prof == nullptr && option(DF_OPT_BWD_OVERLAP) != 0) ? t_side.get() : nullptr;
  cudaStream_t s_dq = s;
  if (sd) {
    // fork after everything already queued on `s`, join back into `s`: callers see ordinary stream semantics
    if (check_cuda(cudaEventRecord(sd->fork, s)) != DF_OK || check_cuda(cudaStreamWaitEvent(sd->stream, sd->fork, 0)) != DF_OK)
      return DF_ERR_CUDA;
    s_dq = sd->stream;
  }
  if (prof && check_cuda(cudaEventRecord(prof[0], s)) != DF_OK) return DF_ERR_CUDA;
  // A profiled call launches each kernel kProfileReps times back to back between its events (the results are the
  // same every time): an event pair around a single launch adds several microseconds to a 70-microsecond kernel.
  const int reps = prof ? kProfileReps : 1;
  for (int rep = 0; (fuse || prof) && rep < reps; ++rep) {
    // (a profiled call with ready-made row sums runs its dQ kernel here too, so that the events split the two kernels)
    const cudaError_t e = fuse ? launch_kernel(k_attn_bwd_dq_tf32_d64<true>, grid_q, dim3(kBwdThreads), dq::kSmemTotal, s, pdl,
                                               tmQk, tmGk, tmKk, tmVk, tmKm, tmDQ, tmO, bp, items_q)
                               : launch_kernel(k_attn_bwd_dq_tf32_d64<false>, grid_q, dim3(kBwdThreads), dq::kSmemTotal, s, pdl,
                                               tmQk, tmGk, tmKk, tmVk, tmKm, tmDQ, tmO, bp, items_q);
    note_launch();
#if defined(DF_ATTN_TRACE) && defined(DF_ATTN_TRACE_DQ)
    if (getenv("DF_ATTN_TRACE_DUMP")) {
      static unsigned long long host[2 * 1024];
      cudaDeviceSynchronize();
      cudaMemcpyFromSymbol(host, g_bwd_trace, sizeof(host));
      for (int slot = 0; slot < 2; ++slot)
        for (int ev = 0; ev < 511; ++ev)
          if (host[slot * 1024 + 2 * ev + 1])
            printf("btrace slot %d ev %llu t %llu\n", slot, host[slot * 1024 + 2 * ev], host[slot * 1024 + 2 * ev + 1] - host[1]);
    }
#endif
    if (check_cuda(e) != DF_OK) return DF_ERR_CUDA;
  }
  if (prof && check_cuda(cudaEventRecord(prof[1], s)) != DF_OK) return DF_ERR_CUDA;
  for (int rep = 0; rep < reps; ++rep) {
    const cudaError_t e = launch_kernel(k_attn_bwd_dkdv_tf32_d64<DF_KV_NSUB>, grid_kv, dim3(kKvThreads), kv::kSmemTotal, s, pdl, tmKk, tmVk,
                                        tmQk, tmGk, tmQm, tmGm, tmDK, tmDV, bp, items_kv);
    note_launch();
#if defined(DF_ATTN_TRACE) && !defined(DF_ATTN_TRACE_DQ)
    if (getenv("DF_ATTN_TRACE_DUMP")) {
      static unsigned long long host[2 * 1024];
      cudaDeviceSynchronize();
      cudaMemcpyFromSymbol(host, g_bwd_trace, sizeof(host));
      for (int slot = 0; slot < 2; ++slot)
        for (int ev = 0; ev < 511; ++ev)
          if (host[slot * 1024 + 2 * ev + 1])
            printf("btrace slot %d ev %llu t %llu\n", slot, host[slot * 1024 + 2 * ev], host[slot * 1024 + 2 * ev + 1] - host[1]);
    }
#endif
    if (check_cuda(e) != DF_OK) return DF_ERR_CUDA;
  }
  if (!fuse && !prof) {
    // with ready-made row sums the dQ kernel is independent of the dK/dV kernel
    const cudaError_t e = launch_kernel(k_attn_bwd_dq_tf32_d64<false>, grid_q, dim3(kBwdThreads), dq::kSmemTotal, s_dq,
                                        pdl && !sd, tmQk, tmGk, tmKk, tmVk, tmKm, tmDQ, tmO, bp, items_q);
    note_launch();
    if (check_cuda(e) != DF_OK) return DF_ERR_CUDA;
  }
  if (prof && check_cuda(cudaEventRecord(prof[2], s)) != DF_OK) return DF_ERR_CUDA;
  if (sd) {
    if (check_cuda(cudaEventRecord(sd->join, sd->stream)) != DF_OK || check_cuda(cudaStreamWaitEvent(s, sd->join, 0)) != DF_OK)
      return DF_ERR_CUDA;
  }
  return DF_OK;
}

}  // namespace df
