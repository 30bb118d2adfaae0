"""Sequence-parallel ring attention on CPU ranks (gloo, world_size 2, 4 and 8): the schedule, the
message flow and the logsumexp merge, with the block arithmetic supplied by the CPU oracle.
The CUDA backend of the same driver is covered by the GPU tests."""
import math
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _ring_module():
    from __graft_entry__ import load_package
    load_package()
    import importlib
    return importlib.import_module("dark_forest_b200.ring")


def test_schedule_covers_every_visible_block_exactly_once():
    ring = _ring_module()
    for world in (1, 2, 3, 4, 8):
        for layout in ("contiguous", "zigzag"):
            n_chunks = world * len(ring.owned_chunks(0, world, layout))
            seen = set()
            per_hop_work = []
            for r in range(world):
                mine = ring.owned_chunks(r, world, layout)
                work = []
                for src, ops in ring.ring_schedule(r, world, layout, True):
                    theirs = ring.owned_chunks(src, world, layout)
                    units = 0.0
                    for op in ops:
                        a, c = mine[op.q_slot], theirs[op.k_slot]
                        assert (a, c) not in seen and c <= a and op.diagonal == (a == c)
                        seen.add((a, c))
                        units += 0.5 if op.diagonal else 1.0
                    work.append(units)
                per_hop_work.append(work)
            assert seen == {(a, c) for a in range(n_chunks) for c in range(a + 1)}
            if layout == "zigzag":  # balanced: the same work on every rank at every hop
                assert all(w == per_hop_work[0] for w in per_hop_work)
    perm = ring.zigzag_permutation(16, 2)
    assert perm == [0, 1, 2, 3, 12, 13, 14, 15, 4, 5, 6, 7, 8, 9, 10, 11]


class OracleBackend:
    """Block arithmetic for CPU tensors (test stand-in for the CUDA backend)."""

    def __init__(self, oracle, H, scale):
        self.o, self.H, self.scale = oracle, H, scale

    def fwd_block(self, q, k, v, out, lse, diagonal):
        o, l = self.o.forward(q.numpy(), k.numpy(), v.numpy(), self.H, self.scale, diagonal)
        out.numpy()[...] = o
        lse.numpy()[...] = l

    def merge(self, o_a, lse_a, o_b, lse_b):
        o, l = self.o.merge_partials(o_a.numpy(), lse_a.numpy(), o_b.numpy(), lse_b.numpy(), self.H)
        o_a.numpy()[...] = o
        lse_a.numpy()[...] = l

    def delta(self, out, d_out, delta):
        delta.numpy()[...] = self.o.delta(np.ascontiguousarray(out.numpy()), np.ascontiguousarray(d_out.numpy()), self.H)

    def bwd_block(self, q, k, v, d_out, lse, delta, d_q, d_k, d_v, diagonal):
        B, C, dm = q.shape
        H, D = self.H, dm // self.H

        def heads(x):
            return x.numpy().reshape(B, -1, H, D).transpose(0, 2, 1, 3).astype(np.float64)

        qh, kh, vh, gh = heads(q), heads(k), heads(v), heads(d_out)
        s = np.einsum("bhid,bhjd->bhij", qh, kh) * self.scale
        if diagonal:
            s = np.where(np.tril(np.ones((C, C), bool)), s, -np.inf)
        p = np.exp(s - lse.numpy().astype(np.float64)[..., None])
        dp = np.einsum("bhid,bhjd->bhij", gh, vh)
        ds = p * (dp - delta.numpy().astype(np.float64)[..., None])

        def flat(x):
            return x.transpose(0, 2, 1, 3).reshape(B, -1, dm).astype(np.float32)

        d_q.numpy()[...] = flat(np.einsum("bhij,bhjd->bhid", ds, kh) * self.scale)
        d_k.numpy()[...] = flat(np.einsum("bhij,bhid->bhjd", ds, qh) * self.scale)
        d_v.numpy()[...] = flat(np.einsum("bhij,bhid->bhjd", p, gh))

    def accumulate(self, dst, src):
        dst.add_(src)


def _worker(rank, world, port, layout, S, H, D, result_dir):
    import torch
    import torch.distributed as dist
    from oracle.attn_oracle import Oracle
    ring = _ring_module()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = Oracle()
        orc.set_threads(1)
        scale = 1.0 / math.sqrt(D)
        q, k, v, go = (orc.fill_normal((1, S, H * D), 0xD1, st) for st in range(4))
        if layout == "zigzag":
            rows = np.array(ring.zigzag_permutation(S, world))
        else:
            rows = np.arange(S)
        L = S // world
        mine = rows[rank * L:(rank + 1) * L]
        tq, tk, tv, tg = (torch.from_numpy(np.ascontiguousarray(x[:, mine])) for x in (q, k, v, go))
        ra = ring.RingAttention(OracleBackend(orc, H, scale), L, H, D, "cpu", causal=True, layout=layout)
        out = torch.empty_like(tq)
        lse = torch.empty((1, H, L))
        ra.forward(tq, tk, tv, out, lse)
        dq, dk, dv = torch.empty_like(tq), torch.empty_like(tq), torch.empty_like(tq)
        ra.backward(tq, tk, tv, out, tg, lse, dq, dk, dv)
        # a second call reuses every buffer: results must not change
        out2, lse2 = torch.empty_like(tq), torch.empty((1, H, L))
        ra.forward(tq, tk, tv, out2, lse2)
        assert torch.equal(out, out2) and torch.equal(lse, lse2)
        o_ref, lse_ref = orc.forward(q, k, v, H, scale, True)
        g_ref = orc.backward(q, k, v, go, H, scale, True)
        err = {"out": float(np.abs(out.numpy() - o_ref[:, mine]).max()),
               "lse": float(np.abs(lse.numpy() - lse_ref[:, :, mine]).max())}
        for name, got, ref in zip(("dq", "dk", "dv"), (dq, dk, dv), g_ref):
            err[name] = float(np.abs(got.numpy() - ref[:, mine]).max())
        np.save(os.path.join(result_dir, f"err_{rank}.npy"), np.array([err[n] for n in ("out", "lse", "dq", "dk", "dv")]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,layout", [(2, "contiguous"), (2, "zigzag"), (4, "zigzag"), (8, "zigzag")])
def test_ring_attention_matches_the_oracle_on_cpu_ranks(tmp_path, world, layout):
    import torch.multiprocessing as mp
    S, H, D = 64 * world, 2, 16
    port = 29600 + world * 7 + (0 if layout == "contiguous" else 3)
    mp.spawn(_worker, args=(world, port, layout, S, H, D, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err = np.load(tmp_path / f"err_{r}.npy")
        assert err.max() <= 5e-5, (r, err)
