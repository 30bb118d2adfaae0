// sm100_ptx.cuh — thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention
// kernels use: mbarriers with bounded waits, TMA tiled loads/stores, tensor memory (TMEM)
// allocation and access, tcgen05 MMA issue/commit, and the shared-memory / instruction
// descriptor encodings.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace df {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Polls three barriers with one round trip to shared memory (the three polls are issued back to back and combined
// afterwards); bit i of the result is set when phase `pi` of barrier i has completed. Never blocks. The
// MMA-issuing warp of a kernel uses it: each of its polls otherwise costs a full shared-memory round trip, in
// series, while the tensor pipe it feeds runs dry.
__device__ __forceinline__ uint32_t mbar_test3(uint32_t b0, uint32_t p0, uint32_t b1, uint32_t p1, uint32_t b2, uint32_t p2) {
  uint32_t m;
  asm volatile(
      "{\n\t.reg .pred pa, pb, pc;\n\t.reg .b32 x, y, z;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pa, [%1], %2;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pb, [%3], %4;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 pc, [%5], %6;\n\t"
      "selp.b32 x, 1, 0, pa;\n\t"
      "selp.b32 y, 2, 0, pb;\n\t"
      "selp.b32 z, 4, 0, pc;\n\t"
      "or.b32 x, x, y;\n\t"
      "or.b32 %0, x, z;\n\t}"
      : "=r"(m)
      : "r"(b0), "r"(p0), "r"(b1), "r"(p1), "r"(b2), "r"(p2)
      : "memory");
  return m;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait. Every wait in the kernels goes through here: it gives up when the CTA's abort
// flag is raised by another thread, after kWaitBudgetNs of wall time, or after a hard number of
// polls, whichever comes first. On giving up it raises the abort flag so that every other role
// of the CTA leaves its loops too, and the caller unwinds to the common teardown.
constexpr uint64_t kWaitBudgetNs = 2000000000ull;  // 2 s: far above any legitimate wait
constexpr uint32_t kWaitMaxPolls = 1u << 28;

// The polling loop lives in ONE out-of-line copy per kernel: inlined at every wait site it added some thirty
// instructions to loops whose speed depends on staying inside the instruction cache.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint64_t budget_ns) {
  const uint64_t t0 = global_timer_ns();
  for (uint32_t polls = 1; polls < kWaitMaxPolls; ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 255u) == 0u) {
      if (*abort_flag != 0u) return false;
      if (global_timer_ns() - t0 > budget_ns) break;
    }
  }
  *abort_flag = 1u;
  return false;
}
// INLINE = true keeps the loop at the wait site: the persistent forward runs short sequences 4 % faster that way
// (the out-of-line call makes it spill), and everything else 2-6 % slower.
template <bool INLINE>
__device__ __forceinline__ bool mbar_wait_sel(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint64_t budget_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  if constexpr (INLINE) {
    const uint64_t t0 = global_timer_ns();
    for (uint32_t polls = 1; polls < kWaitMaxPolls; ++polls) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((polls & 255u) == 0u) {
        if (*abort_flag != 0u) return false;
        if (global_timer_ns() - t0 > budget_ns) break;
      }
    }
    *abort_flag = 1u;
    return false;
  } else {
    return mbar_wait_slow(bar, parity, abort_flag, budget_ns);
  }
}
__device__ __forceinline__ bool mbar_wait_budget(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                 uint64_t budget_ns) {
  return mbar_wait_sel<false>(bar, parity, abort_flag, budget_ns);
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag) {
  return mbar_wait_budget(bar, parity, abort_flag, kWaitBudgetNs);
}

// One lane of a converged warp (all 32 lanes must execute this). The MMA-issuing warp of a kernel runs its role
// with ALL lanes, warp-uniformly, and only guards the tcgen05.mma / tcgen05.commit instructions with this: inside an
// `if (lane == 0)` region instead, every operand is a per-thread value and the issue of one MMA cost 60-85 cycles of
// the thread's own instructions (more when the warp shares its scheduler with busy softmax warps), which bounded a
// 128x64x8 TF32 MMA to half the tensor pipe's rate; written this way 16 N=128 + 32 N=64 MMAs issue in 2.1 K cycles,
// the pipe's full rate, alone or next to eight busy warps (measured with a probe kernel on the B200).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

// Bounded wait and barrier poll for a role that all 32 lanes of a warp run together: every lane gets the same answer,
// so the lanes leave their loops together (a lane that gave up alone would leave the others waiting for it at the
// next elect.sync).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
}
__device__ __forceinline__ uint32_t mbar_test3_warp(uint32_t b0, uint32_t p0, uint32_t b1, uint32_t p1, uint32_t b2, uint32_t p2) {
  return __reduce_and_sync(0xffffffffu, mbar_test3(b0, p0, b1, p1, b2, p2));
}

// ------------------------------------------------------------------ untiled bulk copy
// Global -> shared through the copy engine; completion is counted in bytes on an mbarrier of this CTA. Both addresses
// must be 16-byte aligned and the size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// ------------------------------------------------------------------ proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------ programmatic dependent launch
// pdl_trigger: lets the next kernel of the stream (when it was launched with programmatic stream
// serialization) start its CTAs as soon as SMs free up, instead of after this grid has drained.
// pdl_wait: blocks until every kernel this one depends on has completed and its writes are visible;
// a no-op in a kernel that was launched the ordinary way. Every kernel of the library executes
// pdl_wait in all threads before its first access to global memory.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ------------------------------------------------------------------ TMA (tiled, no multicast)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 4-D tiled load global -> shared, completion counted in bytes on an mbarrier.
// c0 (innermost) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *m, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2, int32_t c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 4-D tiled store shared -> global (bulk async-group completion). Coordinates must be >= 0.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *m, uint32_t src, int32_t c0,
                                             int32_t c1, int32_t c2, int32_t c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 2-D variants (plain row-major matrices: c0 = column, c1 = row)
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *m, uint32_t bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *m, uint32_t src, int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
// Waits until at most one committed store group has not yet read its shared-memory source.
__device__ __forceinline__ void tma_store_wait_read_1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// Waits only until the committed stores have read their shared-memory source (enough before the
// source is overwritten or the CTA exits; the global writes complete with the grid at the latest).
__device__ __forceinline__ void tma_store_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ------------------------------------------------------------------ TMEM
// Allocation is warp-collective; ncols is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread = lane).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------ MMA
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same instructions with the shared-memory descriptor given as its two 32-bit halves (the address lives in the
// low word, everything else in the high word is the same for all K-steps of a tile) and, for *_acc, the accumulate
// flag fixed to 1: an MMA batch written with these and with its low words precomputed in registers is nothing but
// tcgen05.mma instructions, which is what lets the issuing warp keep the tensor pipe fed while it shares its
// scheduler with busy softmax warps (measured with a probe: 16 N=128 + 32 N=64 MMAs next to 16 busy warps in 2155
// cycles this way, 2856 with an address add and an election per MMA; the pipe needs 2048).
__device__ __forceinline__ void mma_tf32_ts_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_ts_lohi_acc(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                                     uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.eq.u32 p, 1, 1;\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ts_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Make an mbarrier track completion of every tcgen05 async op this thread issued so far.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// tcgen05.commit by the elected lane of a warp that runs its MMA role with all lanes (see elect_one)
__device__ __forceinline__ void commit_elected(uint32_t bar) {
  if (elect_one()) mma_commit(bar);
}

// ------------------------------------------------------------------ descriptors
// Instruction descriptor (32 bit) for kind::tf32 / kind::f16 with fp32 accumulation.
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format  (0 f16, 1 bf16, 2 tf32)
//   [15] A major (0 = K, 1 = MN)   [16] B major   [17,23) N >> 3   [24,29) M >> 4
enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2 };
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t M, uint32_t N,
                                                  uint32_t a_mn_major, uint32_t b_mn_major) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Shared-memory matrix descriptor (64 bit).
//   [0,14) start address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) version = 1 (Blackwell)   [61,64) layout type
// Layout types used here:
//   kSwz128      128-byte swizzle, 16-byte atoms (TMA SWIZZLE_128B): 16-byte chunk index XOR (row % 8).
//   kSwz128B32   128-byte swizzle, 32-byte atoms (TMA SWIZZLE_128B_ATOM_32B): 32-byte chunk index
//                XOR (row % 4). The only layout a 32-bit (TF32) MN-major operand may use.
// K-major operand (rows of 128 B along K): SBO = distance between 8-row groups (1024 B when
//   dense), LBO unused (1).
// MN-major operand (rows of 128 B along M/N, one row per K index): LBO = distance between
//   consecutive 128-byte chunks along M/N; SBO = distance between consecutive groups of K rows
//   (8 rows = 1024 B for kSwz128, 4 rows = 512 B for kSwz128B32 when dense).
enum : uint32_t { kSwz128 = 2, kSwz128B32 = 1 };
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type) {
  const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
  const uint32_t hi = (sbo_bytes >> 4) | (1u << 14) | (layout_type << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  return make_smem_desc(smem_addr, lbo_bytes, sbo_bytes, kSwz128);
}

// fp32 -> TF32, round to nearest with ties away from zero (what cvt.rna.tf32.f32 returns, low 13 bits zero), done
// with two integer instructions: the conversion instruction shares the transcendental unit with ex2, which the
// softmax phases of these kernels keep busy, and the integer pipe is idle there.
__device__ __forceinline__ uint32_t cvt_rna_tf32(float x) {
  return (__float_as_uint(x) + 0x1000u) & 0xffffe000u;
}
// The same rounding for a value that only feeds a kind::tf32 MMA as a tensor-memory operand: the MMA ignores the low
// 13 mantissa bits, so adding half a TF32 ulp is all that is needed (one instruction).
__device__ __forceinline__ uint32_t tf32_rna_operand(float x) {
  return __float_as_uint(x) + 0x1000u;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace ptx

// Host side: cuTensorMapEncodeTiled resolved through the runtime (no libcuda link dependency).
typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                    const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
PFN_encodeTiled get_encode_tiled();

// Kernel launch with or without programmatic stream serialization (see pdl_wait above).
template <class... KArgs, class... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl,
                                 Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Tensor map over a [B][S][H*D] tensor viewed as (d, h, s, b): one box = 128 bytes of dims x `rows`
// rows of one head = one 128-byte-wide shared-memory slab. fp32 tensors are typed TFLOAT32, so
// the copy engine rounds fp32 to TF32 (nearest even) while loading; bf16 tensors are copied as
// they are. `b32_atoms` selects the 128-byte swizzle with 32-byte atoms that an MN-major TF32 MMA
// operand needs; otherwise the plain 128-byte swizzle.
// `for_store` types an fp32 tensor FLOAT32, so that a store moves the words unchanged.
inline bool encode_head_tile_map(CUtensorMap *m, const void *base, bool bf16, uint32_t D, uint32_t B, uint32_t H,
                                 uint32_t S, uint32_t rows, bool b32_atoms, bool for_store = false) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return false;
  const cuuint64_t elt = bf16 ? 2 : 4;
  const cuuint64_t dims[4] = {D, H, S, B};
  const cuuint64_t strides[3] = {(cuuint64_t)D * elt, (cuuint64_t)H * D * elt, (cuuint64_t)S * H * D * elt};
  const cuuint32_t box[4] = {(cuuint32_t)(128 / elt), 1, rows, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType ty = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : (for_store ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32);
  const CUresult r = enc(m, ty, 4,
                         const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         b32_atoms ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tensor map over a row-major [rows, cols] fp32 matrix: one box = 128 bytes (32 floats) of a row x `box_rows`
// rows = one 128-byte-swizzled shared-memory slab. Loads are typed TFLOAT32 (fp32 rounded to TF32, nearest
// even, in flight), stores FLOAT32 (words unchanged). Reads outside the matrix give zeros, writes outside are dropped.
inline bool encode_matrix_map(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows, bool for_store) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {32, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(m, for_store ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 2,
                         const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace df
