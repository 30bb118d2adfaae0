/*
 * darkforest_ring.h - C ABI of the sequence-parallel ring attention (library libdarkforest_ring).
 *
 * An optional second library: it links NCCL and libdarkforest_kernels, so single-GPU users of
 * darkforest_kernels.h need no NCCL. None of these symbols has a counterpart in the reference, whose
 * attention is single-GPU and whose only distributed code is a CPU ring all-reduce over TCP
 * (darkforest-core/src/cluster/transport.rs:16-22, cluster/collectives.rs:32-117); a host that wants
 * sequences too long for one GPU binds these next to its launch_fused_* bindings.
 *
 * One process (or thread) per GPU, each with its own handle; a handle is used by one thread at a
 * time. Every rank owns `local_len` rows of Q, K, V, O, dO and the gradients ([local_len, H*D], fp32
 * or bf16, batch 1) and `local_len` columns of lse ([H, local_len] fp32). K/V blocks travel with
 * ncclSend/ncclRecv into the caller's workspace on this GPU; nothing is loaded from a peer's memory.
 * The calls are asynchronous on `stream` (transfers run on a stream the handle owns) and allocate
 * nothing: streams and events are created by df_ring_create, staging memory is the caller's
 * workspace of df_ring_workspace_bytes() bytes, 256-byte aligned, passed to every call.
 */
#ifndef DARKFOREST_RING_H
#define DARKFOREST_RING_H

#include <stddef.h>
#include <stdint.h>

#include "darkforest_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct df_ring df_ring_t;

#define DF_RING_UNIQUE_ID_BYTES 128
/* Row ownership. CONTIGUOUS: rank r owns rows [r L, (r+1) L) and the schedule follows that order (under a
 * causal mask the last rank does W times the work of the first). ZIGZAG: the caller already holds chunks r
 * and 2W-1-r (L/2 rows each, back to back), which gives every rank the same work on every hop. BALANCED: the
 * caller holds contiguous rows; each call moves its tensors into the zigzag order with one grouped send/recv
 * exchange, runs the zigzag schedule and moves the results back. */
#define DF_RING_LAYOUT_CONTIGUOUS 0
#define DF_RING_LAYOUT_ZIGZAG 1
#define DF_RING_LAYOUT_BALANCED 2

/* Rank 0 creates the id and hands it to every rank by the host's own means (a file, a socket, MPI, a store). */
DF_API int df_ring_unique_id(void *id_out /* DF_RING_UNIQUE_ID_BYTES */);

/* Collective over all ranks: builds a non-blocking NCCL communicator and this rank's streams and events.
 * timeout_ms bounds every wait on the host inside this library (0: 30 s): if the communicator is not up by then
 * (a rank that never calls), it is aborted and DF_ERR_RING_TIMEOUT is returned; the same limit applies to the
 * enqueue of every exchange later. bf16 != 0: tensors hold bf16 (d_head 64 or 128), partial results and the
 * travelling accumulators stay fp32. */
DF_API int df_ring_create(df_ring_t **out, const void *unique_id, int rank, int world, int layout, uint32_t n_heads,
                   uint32_t local_len, uint32_t d_head, int bf16, float scale, int causal, uint32_t timeout_ms);
DF_API uint64_t df_ring_workspace_bytes(const df_ring_t *ring);

/* out [L, H*D] and lse [H, L] of this rank's rows. */
DF_API int df_ring_forward(df_ring_t *ring, const void *q, const void *k, const void *v, void *out, float *lse,
                    void *workspace, uint64_t workspace_bytes, void *stream);
/* Gradients of this rank's rows from the saved out and lse. The dK/dV accumulators follow their K/V block round
 * the ring in fp32 and come home after the last hop. */
DF_API int df_ring_backward(df_ring_t *ring, const void *q, const void *k, const void *v, const void *out,
                     const void *d_out, const float *lse, void *d_q, void *d_k, void *d_v, void *workspace,
                     uint64_t workspace_bytes, void *stream);

/* Waits on the host until `stream` and the handle's transfer stream have drained, polling the communicator for
 * asynchronous errors, for at most timeout_ms (0: the handle's limit). When the limit passes (a peer is gone) the
 * communicator is aborted - its kernels then leave the GPU - and DF_ERR_RING_TIMEOUT is returned; the handle
 * refuses further calls. */
DF_API int df_ring_wait(df_ring_t *ring, void *stream, uint32_t timeout_ms);
DF_API int df_ring_last_nccl_result(const df_ring_t *ring);  /* the ncclResult_t behind the last DF_ERR_NCCL */
/* Not collective: a rank may leave alone (the communicator is aborted, not negotiated down). */
DF_API int df_ring_destroy(df_ring_t *ring);

/* Host-only view of the schedule: the blocks rank `rank` computes at hop `hop` (while it holds the K/V of rank
 * (rank - hop) mod world), four ints per block: query slot, first key slot, number of key chunks (2: both chunks
 * of the visiting block are fully visible and go into one call), diagonal flag. Returns the number of blocks
 * (at most 3), or -1 for bad arguments. */
DF_API int df_ring_hop_blocks(int rank, int world, int layout, int causal, int hop, int *ops_out /* 12 ints */);

#ifdef __cplusplus
}
#endif
#endif /* DARKFOREST_RING_H */
