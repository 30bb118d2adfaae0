// ring_nccl.cu — sequence-parallel ring attention behind the C ABI (library libdarkforest_ring).
//
// One process per GPU. Every rank owns a slice of the rows of Q, K, V (batch 1). K/V blocks travel
// round the ring with ncclSend/ncclRecv on a communication stream of their own, into THIS rank's
// caller-owned staging buffers (no remote loads, no multicast), while the attention kernels of the
// current hop run on the caller's stream; block results come from the single-GPU entry points of
// libdarkforest_kernels (df_attn_forward_block, df_attn_backward_block and their bf16 twins),
// partial outputs are merged by logsumexp, and in the backward the fp32 dK/dV accumulators follow
// their K/V block round the ring (their hand-off to the next rank overlaps the next hop's kernels).
//
// The reference has no counterpart: its only distributed code is a CPU ring all-reduce over TCP
// (darkforest-core/src/cluster/transport.rs:16-22, cluster/collectives.rs:32-117); the merge is the
// max/exp rescale of its split-K decode reduction (darkforest-cuda/kernels/attention_fused.cu:714-760).
//
// Ownership layouts (a chunk is the unit of the causal mask, C rows):
//   contiguous  rank r owns rows [r L, (r+1) L): one chunk. Under a causal mask the last rank does
//               W times the work of the first.
//   zigzag      rank r owns chunks r and 2W-1-r (C = L/2 each), stored back to back: every rank has
//               the same visible work on every hop. The caller already holds its rows in this order.
//   balanced    the caller holds plain contiguous rows; the ring moves them into the zigzag order
//               with one grouped send/recv exchange, runs the zigzag schedule and moves the results
//               back, all inside the call.
//
// Failure handling: the communicator is non-blocking; every NCCL call is followed by a poll of
// ncclCommGetAsyncError against a wall-clock deadline. When it passes (a peer that never arrives,
// a lost rank) the communicator is aborted, the handle is marked dead and the call returns
// DF_ERR_RING_TIMEOUT; nothing here waits without a limit on the host, and the kernels it launches
// are the single-GPU ones with their own bounded waits.
#include <math.h>
#include <time.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <nccl.h>

#include "../../include/darkforest_kernels.h"
#include "../../include/darkforest_ring.h"

namespace {

constexpr uint64_t kAlign = 256;
inline uint64_t align_up(uint64_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

// ---- schedule -------------------------------------------------------------------------------------
struct BlockOp {
  int q_slot;     // index into this rank's chunk list
  int k_slot;     // first chunk of the visiting block
  int k_chunks;   // 1, or 2 when both chunks of the visiting block are fully visible (one call over 2C keys)
  int diagonal;   // 1: causal mask inside the block (same global chunk); 0: fully visible
};

int owned_chunks(int rank, int world, int zigzag, int out[2]) {
  if (!zigzag) {
    out[0] = rank;
    return 1;
  }
  out[0] = rank;
  out[1] = 2 * world - 1 - rank;
  return 2;
}

// Blocks that `rank` computes while it holds the K/V of `src`: key chunk c is fully visible to query
// chunk a when c < a, causally masked when c == a, skipped when c > a. Two fully visible key chunks
// of one query chunk are merged into one call (they lie back to back in the visiting block).
int hop_blocks(int rank, int src, int world, int zigzag, int causal, BlockOp out[4]) {
  int mine[2], theirs[2];
  const int nq = owned_chunks(rank, world, zigzag, mine), nk = owned_chunks(src, world, zigzag, theirs);
  int n = 0;
  for (int qs = 0; qs < nq; ++qs) {
    int vis[2] = {0, 0};  // 0 skip, 1 full, 2 diagonal
    for (int ks = 0; ks < nk; ++ks) vis[ks] = !causal ? 1 : (theirs[ks] < mine[qs] ? 1 : (theirs[ks] == mine[qs] ? 2 : 0));
    if (nk == 2 && vis[0] == 1 && vis[1] == 1) {
      out[n++] = BlockOp{qs, 0, 2, 0};
      continue;
    }
    for (int ks = 0; ks < nk; ++ks)
      if (vis[ks]) out[n++] = BlockOp{qs, ks, 1, vis[ks] == 2};
  }
  return n;
}

// ---- small kernels ----------------------------------------------------------------------------------
__global__ void k_f32_to_bf16(const float4 *__restrict__ src, uint2 *__restrict__ dst, size_t n4) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = src[i];
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t *>(&a);
    o.y = *reinterpret_cast<const uint32_t *>(&b);
    dst[i] = o;
  }
}
__global__ void k_fill_f32(float *dst, float value, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = value;
}

}  // namespace

struct df_ring {
  ncclComm_t comm = nullptr;
  bool comm_ok = false, dead = false;
  int rank = 0, world = 1, layout = 0, zigzag = 0, n_slots = 1;
  uint32_t H = 0, L = 0, D = 0, C = 0;
  int bf16 = 0, causal = 1;
  float scale = 1.0f;
  uint32_t timeout_ms = 30000;
  size_t dm = 0, elt = 4;
  cudaStream_t comm_stream = nullptr, side_stream = nullptr;
  cudaEvent_t ev_in = nullptr, ev_recv[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr}, ev_fork = nullptr, ev_join = nullptr,
              ev_acc_ready[2] = {nullptr, nullptr}, ev_acc_recv[2] = {nullptr, nullptr}, ev_relayout = nullptr, ev_out = nullptr;
  // workspace offsets (bytes)
  uint64_t off_kv[2], off_acc[2], off_part_o[2], off_part_lse[2], off_lse_c[2], off_delta_c[2], off_acc_out, off_acc_dq,
      off_part_dq[3], off_part_dk[3], off_part_dv[3], off_zz[5], off_zz_grad[3], ws_bytes = 0;
  int last_nccl = 0;
};

namespace {

using clock_type = std::chrono::steady_clock;

int fail_cuda() { return DF_ERR_CUDA; }
#define RING_CUDA(x)                         \
  do {                                       \
    if ((x) != cudaSuccess) return fail_cuda(); \
  } while (0)
#define RING_ST(x)            \
  do {                        \
    const int st__ = (x);     \
    if (st__ != DF_OK) return st__; \
  } while (0)

// Completion of the last NCCL call on a non-blocking communicator, against the handle's deadline.
int nccl_settle(df_ring *r, ncclResult_t res) {
  if (res == ncclSuccess) return DF_OK;
  if (res != ncclInProgress) {
    r->last_nccl = (int)res;
    return DF_ERR_NCCL;
  }
  const auto deadline = clock_type::now() + std::chrono::milliseconds(r->timeout_ms);
  for (;;) {
    ncclResult_t st = ncclSuccess;
    const ncclResult_t q = ncclCommGetAsyncError(r->comm, &st);
    if (q != ncclSuccess) {
      r->last_nccl = (int)q;
      return DF_ERR_NCCL;
    }
    if (st == ncclSuccess) return DF_OK;
    if (st != ncclInProgress) {
      r->last_nccl = (int)st;
      return DF_ERR_NCCL;
    }
    if (clock_type::now() > deadline) {
      // give up: abort the communicator so that nothing of it stays queued, and refuse further calls
      ncclCommAbort(r->comm);
      r->comm = nullptr;
      r->comm_ok = false;
      r->dead = true;
      return DF_ERR_RING_TIMEOUT;
    }
    struct timespec ts = {0, 200000};  // 0.2 ms
    nanosleep(&ts, nullptr);
  }
}

struct Xfer { const void *send; void *recv; size_t bytes; int send_to, recv_from; };

// One grouped exchange on the communication stream; transfers whose peer is this rank become copies.
int ring_exchange(df_ring *r, const std::vector<Xfer> &xs) {
  if (r->world > 1) {
    RING_ST(nccl_settle(r, ncclGroupStart()));
    for (const Xfer &x : xs) {
      if (x.send && x.send_to != r->rank) {
        const ncclResult_t e = ncclSend(x.send, x.bytes, ncclInt8, x.send_to, r->comm, r->comm_stream);
        if (e != ncclSuccess && e != ncclInProgress) { ncclGroupEnd(); r->last_nccl = (int)e; return DF_ERR_NCCL; }
      }
      if (x.recv && x.recv_from != r->rank) {
        const ncclResult_t e = ncclRecv(x.recv, x.bytes, ncclInt8, x.recv_from, r->comm, r->comm_stream);
        if (e != ncclSuccess && e != ncclInProgress) { ncclGroupEnd(); r->last_nccl = (int)e; return DF_ERR_NCCL; }
      }
    }
    RING_ST(nccl_settle(r, ncclGroupEnd()));
  }
  return DF_OK;
}

uint8_t *at(void *ws, uint64_t off) { return static_cast<uint8_t *>(ws) + off; }

void plan_workspace(df_ring *r) {
  uint64_t o = 0;
  auto take = [&](uint64_t bytes) { const uint64_t at_ = o; o += align_up(bytes); return at_; };
  const uint64_t rows_e = (uint64_t)r->L * r->dm * r->elt, rows_f = (uint64_t)r->L * r->dm * 4;
  const uint64_t chunk_f = (uint64_t)r->C * r->dm * 4, stat = (uint64_t)r->H * r->C * 4;
  for (int i = 0; i < 2; ++i) r->off_kv[i] = take(2 * rows_e);
  for (int i = 0; i < 2; ++i) r->off_acc[i] = take(2 * rows_f);
  for (int i = 0; i < 2; ++i) { r->off_part_o[i] = take(chunk_f); r->off_part_lse[i] = take(stat); }
  for (int i = 0; i < 2; ++i) { r->off_lse_c[i] = take(stat); r->off_delta_c[i] = take(stat); }
  r->off_acc_out = take(r->bf16 ? rows_f : 0);
  r->off_acc_dq = take(r->bf16 ? rows_f : 0);
  // one set of partial gradients per block of a hop (at most three: the first hop of the zigzag schedule)
  for (int i = 0; i < 3; ++i) { r->off_part_dq[i] = take(chunk_f); r->off_part_dk[i] = take(rows_f); r->off_part_dv[i] = take(rows_f); }
  const bool bal = r->layout == DF_RING_LAYOUT_BALANCED;
  for (int i = 0; i < 5; ++i) r->off_zz[i] = take(bal ? rows_e : 0);
  for (int i = 0; i < 3; ++i) r->off_zz_grad[i] = take(bal ? rows_e : 0);
  r->ws_bytes = o;
}

// ---- the block arithmetic, through the C ABI of the single-GPU library ------------------------------------
int fwd_block(df_ring *r, const void *q, const void *k, const void *v, float *out_f32_or_native, float *lse, uint32_t sk,
              int diagonal, cudaStream_t s) {
  if (r->bf16)
    return df_attn_forward_bf16(q, k, v, out_f32_or_native, lse, 1, r->H, r->C, sk, r->D, r->scale, diagonal ? 1 : 0, 0, 1, s);
  return df_attn_forward_block(static_cast<const float *>(q), static_cast<const float *>(k), static_cast<const float *>(v),
                               out_f32_or_native, lse, 1, r->H, r->C, sk, r->D, r->scale, diagonal ? 1 : 0, 0, s);
}
int bwd_block(df_ring *r, const void *q, const void *k, const void *v, const void *d_out, const float *lse, const float *delta,
              float *d_q, float *d_k, float *d_v, uint32_t sk, int diagonal, cudaStream_t s) {
  if (r->bf16)
    return df_attn_backward_block_bf16(q, k, v, d_out, lse, delta, d_q, d_k, d_v, 1, r->H, r->C, sk, r->D, r->scale,
                                       diagonal ? 1 : 0, 0, 1, s);
  return df_attn_backward_block(static_cast<const float *>(q), static_cast<const float *>(k), static_cast<const float *>(v),
                                static_cast<const float *>(d_out), lse, delta, d_q, d_k, d_v, 1, r->H, r->C, sk, r->D,
                                r->scale, diagonal ? 1 : 0, 0, s);
}
int to_native(df_ring *r, const float *src, void *dst, size_t n, cudaStream_t s) {
  if (!r->bf16) {
    if (static_cast<const void *>(src) != dst) RING_CUDA(cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyDeviceToDevice, s));
    return DF_OK;
  }
  const size_t n4 = n / 4;  // n = rows * H * D with D a multiple of 64
  const unsigned grid = (unsigned)((n4 + 255) / 256 < 4096 ? (n4 + 255) / 256 : 4096);
  k_f32_to_bf16<<<grid ? grid : 1, 256, 0, s>>>(reinterpret_cast<const float4 *>(src), static_cast<uint2 *>(dst), n4);
  return cudaGetLastError() == cudaSuccess ? DF_OK : DF_ERR_CUDA;
}
// lse [H, L] <-> per-slot [H, C] (strided copies)
int lse_to_slots(df_ring *r, const float *lse, void *ws, cudaStream_t s) {
  for (int sl = 0; sl < r->n_slots; ++sl)
    RING_CUDA(cudaMemcpy2DAsync(at(ws, r->off_lse_c[sl]), (size_t)r->C * 4, lse + (size_t)sl * r->C, (size_t)r->L * 4,
                                (size_t)r->C * 4, r->H, cudaMemcpyDeviceToDevice, s));
  return DF_OK;
}
int slots_to_lse(df_ring *r, void *ws, float *lse, cudaStream_t s) {
  for (int sl = 0; sl < r->n_slots; ++sl)
    RING_CUDA(cudaMemcpy2DAsync(lse + (size_t)sl * r->C, (size_t)r->L * 4, at(ws, r->off_lse_c[sl]), (size_t)r->C * 4,
                                (size_t)r->C * 4, r->H, cudaMemcpyDeviceToDevice, s));
  return DF_OK;
}

// Contiguous <-> zigzag. Chunk j (of 2W, C rows each) lives on rank j / 2 (slot j % 2) in the contiguous order and on
// rank (j < W ? j : 2W-1-j), slot (j < W ? 0 : 1), in the zigzag order. `to_zigzag`: src tensors are contiguous-order.
// Each entry moves one chunk-sized piece (bytes per chunk given) of one tensor; done as one grouped exchange.
struct Piece { const void *src; void *dst; size_t chunk_bytes; };
int relayout(df_ring *r, const std::vector<Piece> &pieces, bool to_zigzag) {
  const int W = r->world, me = r->rank;
  std::vector<Xfer> xs;
  auto zz_owner = [&](int j) { return j < W ? j : 2 * W - 1 - j; };
  auto zz_slot = [&](int j) { return j < W ? 0 : 1; };
  for (const Piece &p : pieces) {
    for (int sl = 0; sl < 2; ++sl) {
      if (to_zigzag) {
        // I hold chunk j = 2 me + sl (slot sl); it belongs to zz_owner(j), slot zz_slot(j)
        const int j_send = 2 * me + sl;
        // I receive, into slot sl, chunk j_recv = (sl == 0 ? me : 2W-1-me) from rank j_recv / 2, who holds it in slot j_recv % 2
        const int j_recv = sl == 0 ? me : 2 * W - 1 - me;
        Xfer x;
        x.send = static_cast<const uint8_t *>(p.src) + (size_t)sl * p.chunk_bytes;
        x.send_to = zz_owner(j_send);
        x.recv = static_cast<uint8_t *>(p.dst) + (size_t)sl * p.chunk_bytes;
        x.recv_from = j_recv / 2;
        x.bytes = p.chunk_bytes;
        if (x.send_to == me) {
          // my own chunk stays here: which of my zigzag slots takes it?
          void *dst = static_cast<uint8_t *>(p.dst) + (size_t)zz_slot(j_send) * p.chunk_bytes;
          if (cudaMemcpyAsync(dst, x.send, p.chunk_bytes, cudaMemcpyDeviceToDevice, r->comm_stream) != cudaSuccess) return DF_ERR_CUDA;
          x.send = nullptr;
        }
        if (x.recv_from == me) x.recv = nullptr;  // covered by the local copy above (from the sender's side)
        xs.push_back(x);
      } else {
        // I hold zigzag slot sl = chunk j_send; it belongs to rank j_send / 2, slot j_send % 2 of the contiguous order
        const int j_send = sl == 0 ? me : 2 * W - 1 - me;
        const int j_recv = 2 * me + sl;  // the chunk my contiguous slot sl wants, held by zz_owner(j_recv) in slot zz_slot(j_recv)
        Xfer x;
        x.send = static_cast<const uint8_t *>(p.src) + (size_t)sl * p.chunk_bytes;
        x.send_to = j_send / 2;
        x.recv = static_cast<uint8_t *>(p.dst) + (size_t)sl * p.chunk_bytes;
        x.recv_from = zz_owner(j_recv);
        x.bytes = p.chunk_bytes;
        if (x.send_to == me) {
          void *dst = static_cast<uint8_t *>(p.dst) + (size_t)(j_send % 2) * p.chunk_bytes;
          if (cudaMemcpyAsync(dst, x.send, p.chunk_bytes, cudaMemcpyDeviceToDevice, r->comm_stream) != cudaSuccess) return DF_ERR_CUDA;
          x.send = nullptr;
        }
        if (x.recv_from == me) x.recv = nullptr;
        xs.push_back(x);
      }
    }
  }
  return ring_exchange(r, xs);
}

int check_call(df_ring *r, const void *ws, uint64_t ws_bytes) {
  if (!r) return DF_ERR_INVALID_ARG;
  if (r->dead) return DF_ERR_RING_TIMEOUT;
  if (!ws || ws_bytes < r->ws_bytes || (reinterpret_cast<uintptr_t>(ws) & 255u)) return DF_ERR_WORKSPACE;
  return DF_OK;
}

// K/V of hop t: the caller's (or re-laid) tensors at hop 0, afterwards the staging buffer that received them
struct KV { const uint8_t *k, *v; };
KV kv_of_hop(df_ring *r, int t, const void *k0, const void *v0, void *ws) {
  if (t == 0) return KV{static_cast<const uint8_t *>(k0), static_cast<const uint8_t *>(v0)};
  const uint8_t *b = at(ws, r->off_kv[(t - 1) & 1]);
  return KV{b, b + (size_t)r->L * r->dm * r->elt};
}
// posts the K/V hand-off of hop t on the communication stream (send hop t's block on, receive hop t+1's)
int post_kv_exchange(df_ring *r, int t, const KV &cur, void *ws) {
  const size_t bytes = (size_t)r->L * r->dm * r->elt;
  if (t == 0) RING_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_in, 0));
  else RING_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_done[(t - 1) & 1], 0));  // the buffer about to be overwritten was read by hop t-1
  uint8_t *dst = at(ws, r->off_kv[t & 1]);
  const int next = (r->rank + 1) % r->world, prev = (r->rank + r->world - 1) % r->world;
  std::vector<Xfer> xs = {Xfer{cur.k, dst, bytes, next, prev}, Xfer{cur.v, dst + bytes, bytes, next, prev}};
  RING_ST(ring_exchange(r, xs));
  RING_CUDA(cudaEventRecord(r->ev_recv[t & 1], r->comm_stream));
  return DF_OK;
}

}  // namespace

extern "C" {

int df_ring_unique_id(void *id_out) {
  if (!id_out) return DF_ERR_INVALID_ARG;
  static_assert(sizeof(ncclUniqueId) == DF_RING_UNIQUE_ID_BYTES, "ncclUniqueId size");
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) return DF_ERR_NCCL;
  memcpy(id_out, &id, sizeof(id));
  return DF_OK;
}

int df_ring_hop_blocks(int rank, int world, int layout, int causal, int hop, int *ops_out) {
  if (rank < 0 || world <= 0 || rank >= world || hop < 0 || hop >= world || !ops_out) return -1;
  BlockOp ops[4];
  const int src = ((rank - hop) % world + world) % world;
  const int n = hop_blocks(rank, src, world, layout != DF_RING_LAYOUT_CONTIGUOUS, causal, ops);
  for (int i = 0; i < n; ++i) {
    ops_out[4 * i] = ops[i].q_slot;
    ops_out[4 * i + 1] = ops[i].k_slot;
    ops_out[4 * i + 2] = ops[i].k_chunks;
    ops_out[4 * i + 3] = ops[i].diagonal;
  }
  return n;
}

int df_ring_create(df_ring_t **out, const void *unique_id, int rank, int world, int layout, uint32_t n_heads,
                   uint32_t local_len, uint32_t d_head, int bf16, float scale, int causal, uint32_t timeout_ms) {
  if (!out) return DF_ERR_INVALID_ARG;
  *out = nullptr;
  if (!unique_id || world <= 0 || rank < 0 || rank >= world || n_heads == 0 || local_len == 0) return DF_ERR_INVALID_ARG;
  if (layout != DF_RING_LAYOUT_CONTIGUOUS && layout != DF_RING_LAYOUT_ZIGZAG && layout != DF_RING_LAYOUT_BALANCED)
    return DF_ERR_INVALID_ARG;
  if (bf16 ? (d_head != 64 && d_head != 128) : (d_head == 0 || d_head > 128)) return DF_ERR_UNSUPPORTED;
  if (layout != DF_RING_LAYOUT_CONTIGUOUS && (local_len % 2)) return DF_ERR_INVALID_ARG;
  if (((uint64_t)n_heads * d_head) % 4) return DF_ERR_UNSUPPORTED;  // rows are moved and converted 16 bytes at a time
  df_ring *r = new (std::nothrow) df_ring();
  if (!r) return DF_ERR_CUDA;
  r->rank = rank; r->world = world; r->layout = layout;
  r->zigzag = layout != DF_RING_LAYOUT_CONTIGUOUS;
  r->n_slots = r->zigzag ? 2 : 1;
  r->H = n_heads; r->L = local_len; r->D = d_head; r->C = local_len / (uint32_t)r->n_slots;
  r->bf16 = bf16 ? 1 : 0; r->causal = causal ? 1 : 0; r->scale = scale;
  r->timeout_ms = timeout_ms ? timeout_ms : 30000;
  r->dm = (size_t)n_heads * d_head;
  r->elt = bf16 ? 2 : 4;
  plan_workspace(r);
  bool ok = cudaStreamCreateWithFlags(&r->comm_stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaStreamCreateWithFlags(&r->side_stream, cudaStreamNonBlocking) == cudaSuccess;
  cudaEvent_t *evs[] = {&r->ev_in, &r->ev_recv[0], &r->ev_recv[1], &r->ev_done[0], &r->ev_done[1], &r->ev_fork, &r->ev_join,
                        &r->ev_acc_ready[0], &r->ev_acc_ready[1], &r->ev_acc_recv[0], &r->ev_acc_recv[1], &r->ev_relayout, &r->ev_out};
  for (cudaEvent_t *e : evs) ok = ok && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    df_ring_destroy(r);
    return DF_ERR_CUDA;
  }
  df_attn_init();  // the calling thread's side stream of the block backward, created here rather than inside a hop
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  const ncclResult_t res = ncclCommInitRankConfig(&r->comm, world, id, rank, &cfg);
  r->comm_ok = true;  // the handle exists from here on, even while initialisation is in progress
  const int st = nccl_settle(r, res);
  if (st != DF_OK) {
    df_ring_destroy(r);
    return st;
  }
  *out = r;
  return DF_OK;
}

uint64_t df_ring_workspace_bytes(const df_ring_t *r) { return r ? r->ws_bytes : 0; }
int df_ring_last_nccl_result(const df_ring_t *r) { return r ? r->last_nccl : 0; }

int df_ring_wait(df_ring_t *r, void *stream, uint32_t timeout_ms) {
  if (!r) return DF_ERR_INVALID_ARG;
  if (r->dead) return DF_ERR_RING_TIMEOUT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto deadline = clock_type::now() + std::chrono::milliseconds(timeout_ms ? timeout_ms : r->timeout_ms);
  for (;;) {
    const cudaError_t a = cudaStreamQuery(s), b = cudaStreamQuery(r->comm_stream);
    if (a == cudaSuccess && b == cudaSuccess) return DF_OK;
    if ((a != cudaSuccess && a != cudaErrorNotReady) || (b != cudaSuccess && b != cudaErrorNotReady)) return DF_ERR_CUDA;
    if (r->comm) {
      ncclResult_t st = ncclSuccess;
      if (ncclCommGetAsyncError(r->comm, &st) != ncclSuccess || (st != ncclSuccess && st != ncclInProgress)) {
        r->last_nccl = (int)st;
        return DF_ERR_NCCL;
      }
    }
    if (clock_type::now() > deadline) {
      // a peer is gone or stuck: abort the communicator (its kernels then leave), refuse further calls
      if (r->comm) ncclCommAbort(r->comm);
      r->comm = nullptr;
      r->comm_ok = false;
      r->dead = true;
      return DF_ERR_RING_TIMEOUT;
    }
    struct timespec ts = {0, 200000};
    nanosleep(&ts, nullptr);
  }
}

int df_ring_destroy(df_ring_t *r) {
  if (!r) return DF_OK;
  if (r->comm && r->comm_ok) {
    // queued transfers belong to calls that have returned: let them finish, then drop the communicator
    if (!r->dead) {
      cudaStreamSynchronize(r->comm_stream);
      ncclCommAbort(r->comm);  // abort frees without the collective handshake of ncclCommDestroy: a rank may leave alone
    }
  }
  cudaEvent_t evs[] = {r->ev_in, r->ev_recv[0], r->ev_recv[1], r->ev_done[0], r->ev_done[1], r->ev_fork, r->ev_join,
                       r->ev_acc_ready[0], r->ev_acc_ready[1], r->ev_acc_recv[0], r->ev_acc_recv[1], r->ev_relayout, r->ev_out};
  for (cudaEvent_t e : evs)
    if (e) cudaEventDestroy(e);
  if (r->comm_stream) cudaStreamDestroy(r->comm_stream);
  if (r->side_stream) cudaStreamDestroy(r->side_stream);
  delete r;
  return DF_OK;
}

int df_ring_forward(df_ring_t *r, const void *q, const void *k, const void *v, void *out, float *lse, void *workspace,
                    uint64_t workspace_bytes, void *stream) {
  RING_ST(check_call(r, workspace, workspace_bytes));
  if (!q || !k || !v || !out || !lse) return DF_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void *ws = workspace;
  const int W = r->world;
  const size_t chunk_e = (size_t)r->C * r->dm * r->elt;
  const bool bal = r->layout == DF_RING_LAYOUT_BALANCED;
  RING_CUDA(cudaEventRecord(r->ev_in, s));
  const void *q_in = q, *k_in = k, *v_in = v;
  if (bal) {
    RING_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_in, 0));
    std::vector<Piece> pcs = {Piece{q, at(ws, r->off_zz[0]), chunk_e}, Piece{k, at(ws, r->off_zz[1]), chunk_e},
                              Piece{v, at(ws, r->off_zz[2]), chunk_e}};
    RING_ST(relayout(r, pcs, true));
    RING_CUDA(cudaEventRecord(r->ev_relayout, r->comm_stream));
    RING_CUDA(cudaStreamWaitEvent(s, r->ev_relayout, 0));
    RING_CUDA(cudaEventRecord(r->ev_in, s));  // hop 0's hand-off waits for the re-laid tensors through the stream order anyway
    q_in = at(ws, r->off_zz[0]); k_in = at(ws, r->off_zz[1]); v_in = at(ws, r->off_zz[2]);
  }
  // accumulation target of O: fp32 (the caller's tensor when it is fp32 and not re-laid, else workspace)
  float *acc = r->bf16 ? reinterpret_cast<float *>(at(ws, r->off_acc_out))
                       : (bal ? reinterpret_cast<float *>(at(ws, r->off_zz[3])) : static_cast<float *>(out));
  bool started[2] = {false, false};
  for (int t = 0; t < W; ++t) {
    const KV cur = kv_of_hop(r, t, k_in, v_in, ws);
    if (t < W - 1) RING_ST(post_kv_exchange(r, t, cur, ws));
    if (t > 0) RING_CUDA(cudaStreamWaitEvent(s, r->ev_recv[(t - 1) & 1], 0));
    BlockOp ops[4];
    const int src = ((r->rank - t) % W + W) % W;
    const int n = hop_blocks(r->rank, src, W, r->zigzag, r->causal, ops);
    // query slot 0 works on the caller's stream, slot 1 on the side stream: blocks of different query chunks are
    // independent, so the tail of one grid is filled by the other
    bool used_side = false;
    for (int i = 0; i < n; ++i) {
      const BlockOp &op = ops[i];
      cudaStream_t bs = s;
      if (op.q_slot == 1 && n > 1 && ops[0].q_slot != ops[n - 1].q_slot) {
        if (!used_side) {
          RING_CUDA(cudaEventRecord(r->ev_fork, s));
          RING_CUDA(cudaStreamWaitEvent(r->side_stream, r->ev_fork, 0));
          used_side = true;
        }
        bs = r->side_stream;
      }
      const uint8_t *qs = static_cast<const uint8_t *>(q_in) + (size_t)op.q_slot * chunk_e;
      const uint8_t *ks = cur.k + (size_t)op.k_slot * chunk_e, *vs = cur.v + (size_t)op.k_slot * chunk_e;
      float *acc_rows = acc + (size_t)op.q_slot * r->C * r->dm;
      float *lse_c = reinterpret_cast<float *>(at(ws, r->off_lse_c[op.q_slot]));
      const uint32_t sk = r->C * (uint32_t)op.k_chunks;
      if (!started[op.q_slot]) {
        RING_ST(fwd_block(r, qs, ks, vs, acc_rows, lse_c, sk, op.diagonal, bs));
        started[op.q_slot] = true;
      } else {
        float *po = reinterpret_cast<float *>(at(ws, r->off_part_o[op.q_slot]));
        float *pl = reinterpret_cast<float *>(at(ws, r->off_part_lse[op.q_slot]));
        RING_ST(fwd_block(r, qs, ks, vs, po, pl, sk, op.diagonal, bs));
        RING_ST(df_attn_merge_partials(acc_rows, lse_c, po, pl, 1, r->H, r->C, r->D, bs));
      }
    }
    if (used_side) {
      RING_CUDA(cudaEventRecord(r->ev_join, r->side_stream));
      RING_CUDA(cudaStreamWaitEvent(s, r->ev_join, 0));
    }
    RING_CUDA(cudaEventRecord(r->ev_done[t & 1], s));
  }
  for (int sl = 0; sl < r->n_slots; ++sl)
    if (!started[sl]) {  // only without a causal mask... or never: the diagonal block is always visible
      RING_CUDA(cudaMemsetAsync(acc + (size_t)sl * r->C * r->dm, 0, (size_t)r->C * r->dm * 4, s));
      k_fill_f32<<<64, 256, 0, s>>>(reinterpret_cast<float *>(at(ws, r->off_lse_c[sl])), -INFINITY, (size_t)r->H * r->C);
    }
  if (!bal) {
    RING_ST(slots_to_lse(r, ws, lse, s));
    if (r->bf16) RING_ST(to_native(r, acc, out, (size_t)r->L * r->dm, s));  // one rounding to bf16 at the very end
  } else {
    // results back into the caller's contiguous order: O (native dtype) and the per-chunk lse
    void *zz_out = at(ws, r->off_zz[3]);
    if (r->bf16) RING_ST(to_native(r, acc, zz_out, (size_t)r->L * r->dm, s));
    RING_CUDA(cudaEventRecord(r->ev_out, s));
    RING_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_out, 0));
    const size_t stat = (size_t)r->H * r->C * 4;
    // lse chunks travel as [H, C] pieces through the delta slots (free in the forward) and are then spread into [H, L]
    std::vector<Piece> pcs = {Piece{zz_out, out, chunk_e}};
    RING_ST(relayout(r, pcs, false));
    // the two lse slots are separate buffers: move them one piece at a time with the same routing
    {
      const int me = r->rank;
      std::vector<Xfer> xs;
      for (int sl = 0; sl < 2; ++sl) {
        const int j_send = sl == 0 ? me : 2 * W - 1 - me, j_recv = 2 * me + sl;
        Xfer x;
        x.send = at(ws, r->off_lse_c[sl]);
        x.send_to = j_send / 2;
        x.recv = at(ws, r->off_delta_c[sl]);
        x.recv_from = j_recv < W ? j_recv : 2 * W - 1 - j_recv;
        x.bytes = stat;
        if (x.send_to == me) {
          RING_CUDA(cudaMemcpyAsync(at(ws, r->off_delta_c[j_send % 2]), x.send, stat, cudaMemcpyDeviceToDevice, r->comm_stream));
          x.send = nullptr;
        }
        if (x.recv_from == me) x.recv = nullptr;
        xs.push_back(x);
      }
      RING_ST(ring_exchange(r, xs));
    }
    RING_CUDA(cudaEventRecord(r->ev_relayout, r->comm_stream));
    RING_CUDA(cudaStreamWaitEvent(s, r->ev_relayout, 0));
    for (int sl = 0; sl < 2; ++sl)
      RING_CUDA(cudaMemcpy2DAsync(lse + (size_t)sl * r->C, (size_t)r->L * 4, at(ws, r->off_delta_c[sl]), (size_t)r->C * 4,
                                  (size_t)r->C * 4, r->H, cudaMemcpyDeviceToDevice, s));
  }
  return cudaGetLastError() == cudaSuccess ? DF_OK : DF_ERR_CUDA;
}

int df_ring_backward(df_ring_t *r, const void *q, const void *k, const void *v, const void *out, const void *d_out,
                     const float *lse, void *d_q, void *d_k, void *d_v, void *workspace, uint64_t workspace_bytes,
                     void *stream) {
  RING_ST(check_call(r, workspace, workspace_bytes));
  if (!q || !k || !v || !out || !d_out || !lse || !d_q || !d_k || !d_v) return DF_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void *ws = workspace;
  const int W = r->world;
  const size_t chunk_e = (size_t)r->C * r->dm * r->elt, rows_f = (size_t)r->L * r->dm * 4, chunk_n = (size_t)r->C * r->dm;
  const size_t stat = (size_t)r->H * r->C * 4;
  const bool bal = r->layout == DF_RING_LAYOUT_BALANCED;
  const int next = (r->rank + 1) % W, prev = (r->rank + W - 1) % W;
  // row statistics in the caller's order first: delta = rowsum(dO o O) is row-local
  for (int sl = 0; sl < r->n_slots; ++sl) {
    const uint8_t *o_rows = static_cast<const uint8_t *>(out) + (size_t)sl * chunk_e;
    const uint8_t *g_rows = static_cast<const uint8_t *>(d_out) + (size_t)sl * chunk_e;
    float *dl = reinterpret_cast<float *>(at(ws, r->off_delta_c[sl]));
    if (r->bf16) RING_ST(df_attn_delta_bf16(o_rows, g_rows, dl, 1, r->H, r->C, r->D, s));
    else RING_ST(df_attn_delta(reinterpret_cast<const float *>(o_rows), reinterpret_cast<const float *>(g_rows), dl, 1, r->H, r->C, r->D, s));
  }
  RING_ST(lse_to_slots(r, lse, ws, s));
  RING_CUDA(cudaEventRecord(r->ev_in, s));
  const void *q_in = q, *k_in = k, *v_in = v, *g_in = d_out;
  if (bal) {
    RING_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_in, 0));
    std::vector<Piece> pcs = {Piece{q, at(ws, r->off_zz[0]), chunk_e}, Piece{k, at(ws, r->off_zz[1]), chunk_e},
                              Piece{v, at(ws, r->off_zz[2]), chunk_e}, Piece{d_out, at(ws, r->off_zz[4]), chunk_e}};
    RING_ST(relayout(r, pcs, true));
    // statistics: the two slots are separate buffers; they go through the partial-lse buffers and back
    {
      const int me = r->rank;
      for (int which = 0; which < 2; ++which) {
        std::vector<Xfer> xs;
        for (int sl = 0; sl < 2; ++sl) {
          const int j_send = 2 * me + sl, j_recv = sl == 0 ? me : 2 * W - 1 - me;
          const uint64_t *src_off = which ? r->off_delta_c : r->off_lse_c;
          Xfer x;
          x.send = at(ws, src_off[sl]);
          x.send_to = j_send < W ? j_send : 2 * W - 1 - j_send;
          x.recv = at(ws, (which ? r->off_part_o : r->off_part_lse)[sl]);
          x.recv_from = j_recv / 2;
          x.bytes = stat;
          if (x.send_to == me) {
            RING_CUDA(cudaMemcpyAsync(at(ws, (which ? r->off_part_o : r->off_part_lse)[j_send < W ? 0 : 1]), x.send, stat,
                                      cudaMemcpyDeviceToDevice, r->comm_stream));
            x.send = nullptr;
          }
          if (x.recv_from == me) x.recv = nullptr;
          xs.push_back(x);
        }
        RING_ST(ring_exchange(r, xs));
      }
      for (int sl = 0; sl < 2; ++sl) {
        RING_CUDA(cudaMemcpyAsync(at(ws, r->off_lse_c[sl]), at(ws, r->off_part_lse[sl]), stat, cudaMemcpyDeviceToDevice, r->comm_stream));
        RING_CUDA(cudaMemcpyAsync(at(ws, r->off_delta_c[sl]), at(ws, r->off_part_o[sl]), stat, cudaMemcpyDeviceToDevice, r->comm_stream));
      }
    }
    RING_CUDA(cudaEventRecord(r->ev_relayout, r->comm_stream));
    RING_CUDA(cudaStreamWaitEvent(s, r->ev_relayout, 0));
    RING_CUDA(cudaEventRecord(r->ev_in, s));
    q_in = at(ws, r->off_zz[0]); k_in = at(ws, r->off_zz[1]); v_in = at(ws, r->off_zz[2]); g_in = at(ws, r->off_zz[4]);
  }
  // fp32 accumulators: dQ stays here, dK/dV travel with their block
  float *dq_acc = r->bf16 ? reinterpret_cast<float *>(at(ws, r->off_acc_dq))
                          : (bal ? reinterpret_cast<float *>(at(ws, r->off_zz_grad[0])) : static_cast<float *>(d_q));
  RING_CUDA(cudaMemsetAsync(dq_acc, 0, rows_f, s));
  RING_CUDA(cudaMemsetAsync(at(ws, r->off_acc[0]), 0, 2 * rows_f, s));
  for (int t = 0; t < W; ++t) {
    const KV cur = kv_of_hop(r, t, k_in, v_in, ws);
    if (t < W - 1) RING_ST(post_kv_exchange(r, t, cur, ws));
    if (t > 0) RING_CUDA(cudaStreamWaitEvent(s, r->ev_recv[(t - 1) & 1], 0));
    BlockOp ops[4];
    const int src = ((r->rank - t) % W + W) % W;
    const int n = hop_blocks(r->rank, src, W, r->zigzag, r->causal, ops);
    const bool two_streams = n > 1 && ops[0].q_slot != ops[n - 1].q_slot;
    bool used_side = false;
    // block kernels first (they do not need the travelling accumulators) ...
    for (int i = 0; i < n; ++i) {
      const BlockOp &op = ops[i];
      cudaStream_t bs = s;
      const int set = i;
      if (two_streams && op.q_slot == 1) {
        if (!used_side) {
          RING_CUDA(cudaEventRecord(r->ev_fork, s));
          RING_CUDA(cudaStreamWaitEvent(r->side_stream, r->ev_fork, 0));
          used_side = true;
        }
        bs = r->side_stream;
      }
      const uint8_t *qs = static_cast<const uint8_t *>(q_in) + (size_t)op.q_slot * chunk_e;
      const uint8_t *gs = static_cast<const uint8_t *>(g_in) + (size_t)op.q_slot * chunk_e;
      const uint8_t *ks = cur.k + (size_t)op.k_slot * chunk_e, *vs = cur.v + (size_t)op.k_slot * chunk_e;
      const uint32_t sk = r->C * (uint32_t)op.k_chunks;
      float *pdq = reinterpret_cast<float *>(at(ws, r->off_part_dq[set]));
      float *pdk = reinterpret_cast<float *>(at(ws, r->off_part_dk[set]));
      float *pdv = reinterpret_cast<float *>(at(ws, r->off_part_dv[set]));
      RING_ST(bwd_block(r, qs, ks, vs, gs, reinterpret_cast<const float *>(at(ws, r->off_lse_c[op.q_slot])),
                        reinterpret_cast<const float *>(at(ws, r->off_delta_c[op.q_slot])), pdq, pdk, pdv, sk, op.diagonal, bs));
      RING_ST(df_attn_accumulate(dq_acc + (size_t)op.q_slot * chunk_n, pdq, chunk_n, bs));  // same query chunk: same stream
    }
    if (used_side) {
      RING_CUDA(cudaEventRecord(r->ev_join, r->side_stream));
      RING_CUDA(cudaStreamWaitEvent(s, r->ev_join, 0));
    }
    // ... then the block's dK/dV go into the accumulators that arrived with it (hop 0: zeroed above)
    if (t > 0) RING_CUDA(cudaStreamWaitEvent(s, r->ev_acc_recv[t & 1], 0));
    float *acc_k = reinterpret_cast<float *>(at(ws, r->off_acc[t & 1])), *acc_v = acc_k + (size_t)r->L * r->dm;
    for (int i = 0; i < n; ++i) {
      const BlockOp &op = ops[i];
      const int set = i;
      const size_t cnt = chunk_n * (size_t)op.k_chunks, off = (size_t)op.k_slot * chunk_n;
      RING_ST(df_attn_accumulate(acc_k + off, reinterpret_cast<float *>(at(ws, r->off_part_dk[set])), cnt, s));
      RING_ST(df_attn_accumulate(acc_v + off, reinterpret_cast<float *>(at(ws, r->off_part_dv[set])), cnt, s));
    }
    RING_CUDA(cudaEventRecord(r->ev_done[t & 1], s));
    RING_CUDA(cudaEventRecord(r->ev_acc_ready[t & 1], s));
    // hand the accumulators to the next rank; it overlaps the next hop's kernels. After the last hop they
    // arrive at the rank that owns the block.
    if (W > 1) {
      RING_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_acc_ready[t & 1], 0));
      std::vector<Xfer> xs = {Xfer{acc_k, at(ws, r->off_acc[(t + 1) & 1]), 2 * rows_f, next, prev}};
      RING_ST(ring_exchange(r, xs));
      RING_CUDA(cudaEventRecord(r->ev_acc_recv[(t + 1) & 1], r->comm_stream));
    }
  }
  const int fin = W > 1 ? (W & 1) : 0;  // the buffer that received the last hand-off
  if (W > 1) RING_CUDA(cudaStreamWaitEvent(s, r->ev_acc_recv[fin], 0));
  const float *fin_k = reinterpret_cast<const float *>(at(ws, r->off_acc[fin])), *fin_v = fin_k + (size_t)r->L * r->dm;
  const size_t n_rows = (size_t)r->L * r->dm;
  if (!bal) {
    if (r->bf16) RING_ST(to_native(r, dq_acc, d_q, n_rows, s));
    RING_ST(to_native(r, fin_k, d_k, n_rows, s));
    RING_ST(to_native(r, fin_v, d_v, n_rows, s));
  } else {
    void *zq = at(ws, r->off_zz_grad[0]), *zk = at(ws, r->off_zz_grad[1]), *zv = at(ws, r->off_zz_grad[2]);
    // native-dtype zigzag gradients, then home. fp32: dq_acc already sits in zz_grad[0]
    if (r->bf16) RING_ST(to_native(r, dq_acc, zq, n_rows, s));
    RING_ST(to_native(r, fin_k, zk, n_rows, s));
    RING_ST(to_native(r, fin_v, zv, n_rows, s));
    RING_CUDA(cudaEventRecord(r->ev_out, s));
    RING_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_out, 0));
    std::vector<Piece> pcs = {Piece{zq, d_q, chunk_e}, Piece{zk, d_k, chunk_e}, Piece{zv, d_v, chunk_e}};
    RING_ST(relayout(r, pcs, false));
    RING_CUDA(cudaEventRecord(r->ev_relayout, r->comm_stream));
    RING_CUDA(cudaStreamWaitEvent(s, r->ev_relayout, 0));
  }
  return cudaGetLastError() == cudaSuccess ? DF_OK : DF_ERR_CUDA;
}

}  // extern "C"
