"""Sequence-parallel ring attention over the block entry points of the attention library.

The reference has no counterpart (its only distributed code is a CPU ring all-reduce,
darkforest-core/src/cluster/collectives.rs:32-117); the partial-result merge is the same
max/exp rescale as its split-K decode reduction (darkforest-cuda/kernels/attention_fused.cu:714-760).

One process per GPU. Every rank owns a slice of the sequence of Q, K, V (batch 1). K/V blocks
travel round the ring with point-to-point send/recv (NCCL over NVLink on GPUs, gloo in the CPU
tests); each hop's transfer is posted before the hop's attention kernels are launched so that
the copy overlaps the math. Blocks land in this rank's own pre-allocated buffers and are read
from there (no remote loads). Partial outputs are merged by logsumexp. The backward sends the
dK/dV accumulators round the ring together with their K/V block, so that after `world` hops
every accumulator is back on the rank that owns the block.

Two ownership layouts (chunk = the unit of the causal mask):
  "contiguous"  rank r owns rows [r*L, (r+1)*L): one chunk, index r. Simple, but under a causal
                mask rank r has r+1 visible blocks out of `world`: the last rank does all the work.
  "zigzag"      rank r owns chunks r and 2*world-1-r, each L/2 rows, stored back to back. Every
                rank then has the same amount of visible work on every hop (two block-units).
`zigzag_permutation` gives the row order that turns a contiguous sequence into the zigzag layout.

The arithmetic is delegated to a backend: `CudaBackend` calls the C ABI
(df_attn_forward_block / df_attn_backward_block / df_attn_merge_partials / df_attn_accumulate /
df_attn_delta). Tests substitute a CPU backend to exercise the schedule and the message flow
with world_size > 1 and no GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple


def owned_chunks(rank: int, world: int, layout: str) -> List[int]:
    """Global chunk indices owned by `rank`, in storage order."""
    if layout == "contiguous":
        return [rank]
    if layout == "zigzag":
        return [rank, 2 * world - 1 - rank]
    raise ValueError(f"unknown layout {layout!r}")


def zigzag_permutation(seq_len: int, world: int) -> List[int]:
    """Row indices such that x[perm] laid out contiguously over ranks is the zigzag layout."""
    if seq_len % (2 * world):
        raise ValueError("seq_len must be a multiple of 2*world for the zigzag layout")
    c = seq_len // (2 * world)
    perm: List[int] = []
    for r in range(world):
        for chunk in (r, 2 * world - 1 - r):
            perm.extend(range(chunk * c, (chunk + 1) * c))
    return perm


@dataclass(frozen=True)
class BlockOp:
    q_slot: int      # index into this rank's chunk list
    k_slot: int      # index into the visiting rank's chunk list
    diagonal: bool   # True: causal mask inside the block (same global chunk); False: fully visible


def hop_blocks(rank: int, src: int, world: int, layout: str, causal: bool) -> List[BlockOp]:
    """Blocks that `rank` computes while it holds the K/V of `src`: a key chunk c is fully visible
    to a query chunk a when c < a, causally masked when c == a, and skipped when c > a."""
    ops = []
    for qs, a in enumerate(owned_chunks(rank, world, layout)):
        for ks, c in enumerate(owned_chunks(src, world, layout)):
            if not causal:
                ops.append(BlockOp(qs, ks, False))
            elif c < a:
                ops.append(BlockOp(qs, ks, False))
            elif c == a:
                ops.append(BlockOp(qs, ks, True))
    return ops


def ring_schedule(rank: int, world: int, layout: str, causal: bool) -> List[Tuple[int, List[BlockOp]]]:
    """[(src rank whose K/V is held at hop t, blocks to compute)] for t = 0..world-1."""
    return [((rank - t) % world, hop_blocks(rank, (rank - t) % world, world, layout, causal)) for t in range(world)]


class CudaBackend:
    """Block arithmetic on the GPU through the C ABI of this package."""

    def __init__(self, pkg, n_heads: int, scale: float):
        self.pkg, self.H, self.scale = pkg, n_heads, scale

    def fwd_block(self, q, k, v, out, lse, diagonal):
        self.pkg.forward(q, k, v, self.H, self.scale, causal=diagonal, out=out, lse=lse, causal_shift=0)

    def merge(self, o_a, lse_a, o_b, lse_b):
        self.pkg.merge_partials(o_a, lse_a, o_b, lse_b, self.H)

    def delta(self, out, d_out, delta):
        self.pkg.delta(out, d_out, self.H, delta_buf=delta)

    def bwd_block(self, q, k, v, d_out, lse, delta, d_q, d_k, d_v, diagonal):
        self.pkg.backward_block(q, k, v, d_out, lse, delta, self.H, self.scale, causal=diagonal, causal_shift=0,
                                d_q=d_q, d_k=d_k, d_v=d_v)

    def accumulate(self, dst, src):
        self.pkg.accumulate(dst, src)


class CudaBackendBf16:
    """bf16 variant: Q, K, V, dO (and the final O) are bfloat16; every partial result (block outputs,
    gradients) is produced in fp32 so that merging and summing over hops adds no bf16 rounding."""
    io_dtype_name = "bfloat16"

    def __init__(self, pkg, n_heads: int, scale: float):
        self.pkg, self.H, self.scale = pkg, n_heads, scale

    def fwd_block(self, q, k, v, out, lse, diagonal):
        self.pkg.forward_bf16(q, k, v, self.H, self.scale, causal=diagonal, out=out, lse=lse, causal_shift=0, out_fp32=True)

    def merge(self, o_a, lse_a, o_b, lse_b):
        self.pkg.merge_partials(o_a, lse_a, o_b, lse_b, self.H)

    def delta(self, out, d_out, delta):
        self.pkg.delta_bf16(out, d_out, self.H, delta_buf=delta)

    def bwd_block(self, q, k, v, d_out, lse, delta, d_q, d_k, d_v, diagonal):
        self.pkg.backward_block_bf16(q, k, v, d_out, lse, delta, self.H, self.scale, causal=diagonal, causal_shift=0,
                                     d_q=d_q, d_k=d_k, d_v=d_v, out_fp32=True)

    def accumulate(self, dst, src):
        self.pkg.accumulate(dst, src)


class RingAttention:
    """Ring attention for one rank. All buffers are allocated once, here; forward() and
    backward() allocate nothing.

    q, k, v, out, d_out, d_q, d_k, d_v: [1, L, H*D] on `device`, L = local rows, float32 or (with a
    bf16 backend) bfloat16; lse: [1, H, L] float32. With layout "zigzag" the L rows are this rank's
    two chunks back to back. Partial results and the travelling dK/dV accumulators are always fp32.
    """

    def __init__(self, backend, local_len: int, n_heads: int, d_head: int, device, group=None, causal: bool = True,
                 layout: str = "zigzag"):
        import torch
        import torch.distributed as dist
        self.dist, self.torch = dist, torch
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.backend, self.causal, self.layout = backend, causal, layout
        self.H, self.D, self.L = n_heads, d_head, local_len
        self.n_slots = len(owned_chunks(self.rank, self.world, layout))
        if local_len % self.n_slots:
            raise ValueError("local_len must be even for the zigzag layout")
        self.C = local_len // self.n_slots
        self.schedule = ring_schedule(self.rank, self.world, layout, causal)
        self.next = (self.rank + 1) % self.world
        self.prev = (self.rank - 1) % self.world
        dm = n_heads * d_head
        f32 = dict(dtype=torch.float32, device=device)
        self.io_bf16 = getattr(backend, "io_dtype_name", "float32") == "bfloat16"
        io = dict(dtype=torch.bfloat16 if self.io_bf16 else torch.float32, device=device)
        # K and V travel as one message: [2, 1, L, H*D]; two buffers alternate between hops
        self.kv = [torch.empty((2, 1, local_len, dm), **io) for _ in range(2)]
        # fp32 accumulators for O and dQ when the caller's tensors are bf16
        self.acc_out = torch.empty((1, local_len, dm), **f32) if self.io_bf16 else None
        self.acc_dq = torch.empty((1, local_len, dm), **f32) if self.io_bf16 else None
        self.dkv = [torch.empty((2, 1, local_len, dm), **f32) for _ in range(2)]   # travelling dK/dV accumulators
        self.part_o = torch.empty((1, self.C, dm), **f32)                         # per-block partial results
        self.part_lse = torch.empty((1, n_heads, self.C), **f32)
        self.lse_c = [torch.empty((1, n_heads, self.C), **f32) for _ in range(self.n_slots)]
        self.delta_c = [torch.empty((1, n_heads, self.C), **f32) for _ in range(self.n_slots)]
        self.part_dq = torch.empty((1, self.C, dm), **f32)
        self.part_dk = torch.empty((1, self.C, dm), **f32)
        self.part_dv = torch.empty((1, self.C, dm), **f32)

    # ------------------------------------------------------------------ helpers
    def _rows(self, x, slot):
        return x[:, slot * self.C:(slot + 1) * self.C]          # contiguous because batch == 1

    def _exchange(self, send_buf, recv_buf):
        """Post send to the next rank and receive from the previous one; returns the requests."""
        d = self.dist
        if self.world == 1:
            return []
        ops = [d.P2POp(d.isend, send_buf, self.next, self.group), d.P2POp(d.irecv, recv_buf, self.prev, self.group)]
        return d.batch_isend_irecv(ops)

    @staticmethod
    def _wait(reqs):
        for r in reqs:
            r.wait()

    # ------------------------------------------------------------------ forward
    def forward(self, q, k, v, out, lse):
        if q.shape[0] != 1:
            raise ValueError("ring attention handles batch 1 (long sequences); shard batches across GPUs instead")
        W = self.world
        cur = 0
        self.kv[0][0].copy_(k)
        self.kv[0][1].copy_(v)
        acc = self.acc_out if self.io_bf16 else out
        started = [False] * self.n_slots
        for t, (src, blocks) in enumerate(self.schedule):
            reqs = self._exchange(self.kv[cur], self.kv[cur ^ 1]) if t < W - 1 else []
            kbuf, vbuf = self.kv[cur][0], self.kv[cur][1]
            for op in blocks:
                qs = self._rows(q, op.q_slot)
                ks, vs = self._rows(kbuf, op.k_slot), self._rows(vbuf, op.k_slot)
                if not started[op.q_slot]:
                    self.backend.fwd_block(qs, ks, vs, self._rows(acc, op.q_slot), self.lse_c[op.q_slot], op.diagonal)
                    started[op.q_slot] = True
                else:
                    self.backend.fwd_block(qs, ks, vs, self.part_o, self.part_lse, op.diagonal)
                    self.backend.merge(self._rows(acc, op.q_slot), self.lse_c[op.q_slot], self.part_o, self.part_lse)
            self._wait(reqs)
            cur ^= 1 if t < W - 1 else 0
        for slot in range(self.n_slots):
            if not started[slot]:  # cannot happen with a causal mask (the diagonal block is always visible)
                self._rows(acc, slot).zero_()
                self.lse_c[slot].fill_(float("-inf"))
            lse[:, :, slot * self.C:(slot + 1) * self.C].copy_(self.lse_c[slot])
        if self.io_bf16:
            out.copy_(acc)  # one rounding to bf16 at the very end
        return out, lse

    # ------------------------------------------------------------------ backward
    def backward(self, q, k, v, out, d_out, lse, d_q, d_k, d_v):
        W = self.world
        for slot in range(self.n_slots):
            self.lse_c[slot].copy_(lse[:, :, slot * self.C:(slot + 1) * self.C])
            self.backend.delta(self._rows(out, slot), self._rows(d_out, slot), self.delta_c[slot])
        cur = 0
        self.kv[0][0].copy_(k)
        self.kv[0][1].copy_(v)
        dcur = 0
        self.dkv[0].zero_()
        dq_acc = self.acc_dq if self.io_bf16 else d_q
        dq_acc.zero_()
        for t, (src, blocks) in enumerate(self.schedule):
            reqs = self._exchange(self.kv[cur], self.kv[cur ^ 1]) if t < W - 1 else []
            kbuf, vbuf = self.kv[cur][0], self.kv[cur][1]
            dkbuf, dvbuf = self.dkv[dcur][0], self.dkv[dcur][1]
            for op in blocks:
                self.backend.bwd_block(self._rows(q, op.q_slot), self._rows(kbuf, op.k_slot), self._rows(vbuf, op.k_slot),
                                       self._rows(d_out, op.q_slot), self.lse_c[op.q_slot], self.delta_c[op.q_slot],
                                       self.part_dq, self.part_dk, self.part_dv, op.diagonal)
                self.backend.accumulate(self._rows(dq_acc, op.q_slot), self.part_dq)
                self.backend.accumulate(self._rows(dkbuf, op.k_slot), self.part_dk)
                self.backend.accumulate(self._rows(dvbuf, op.k_slot), self.part_dv)
            self._wait(reqs)
            if t < W - 1:
                cur ^= 1
            # the accumulators follow their K/V block; after the last hop they arrive at their owner
            if W > 1:
                self._wait(self._exchange(self.dkv[dcur], self.dkv[dcur ^ 1]))
                dcur ^= 1
        d_k.copy_(self.dkv[dcur][0])
        d_v.copy_(self.dkv[dcur][1])
        if self.io_bf16:
            d_q.copy_(dq_acc)
        return d_q, d_k, d_v
