"""The backward entry point that takes no scratch argument (df_attn_backward_static_scratch).

It serves hosts that cannot allocate at call time and have no buffer to lend, so its delta row
sums live in an array built into the library. This file checks, through the C ABI, that it
returns what df_attn_backward returns with a caller-provided delta buffer: on two calls in a
row (the second on a different, larger problem, so that whatever the first call left in the
shared array would show up if it mattered), and that a problem beyond the array's stated limit
is refused with its own status before anything runs.

The file sorts last so that a run stopping at the first failure has already run everything else;
it also passes when run alone in a fresh process.
"""
import numpy as np
import pytest

import helpers as hp
from helpers import pkg, to_dev

pytestmark = pytest.mark.gpu


def _case(oracle, B, H, S, D, seed):
    return tuple(oracle.fill_normal((B, S, H * D), seed, st) for st in range(4))


def test_static_scratch_backward_matches_the_regular_entry_point_twice_in_a_row(oracle):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    p = pkg()
    for call, (B, H, S, D) in enumerate([(2, 3, 200, 64), (1, 12, 640, 64), (1, 2, 77, 32)]):
        q, k, v, go = _case(oracle, B, H, S, D, 900 + call)
        tq, tk, tv, tg = to_dev(q, k, v, go)
        scale = hp.default_scale(D)
        out, lse = p.forward(tq, tk, tv, H, scale, True)
        ref = p.backward(tq, tk, tv, out, tg, lse, H, scale, True)
        got = p.backward_static_scratch(tq, tk, tv, out, tg, lse, H, scale, True)
        assert p.sync_status() == 0
        tol = hp.TOL_GRAD_REL_TF32 if D == 64 else hp.TOL_GRAD_REL_FP32
        for g, r, name in zip(got, ref, ("dq", "dk", "dv")):
            assert hp.rel_err(g.cpu().numpy(), r.cpu().numpy()) <= tol, (call, name)
        # and both agree with the CPU oracle
        for g, r in zip(got, oracle.backward(q, k, v, go, H, scale, True)):
            assert hp.rel_err(g.cpu().numpy(), r) <= tol, call


def test_static_scratch_backward_leaves_device_memory_untouched(oracle):
    """The promise in the entry point's name, measured: with the gradient tensors supplied by the caller and
    one call already made on this device (the first call looks up the array's address), a further call
    changes neither the driver's count of free device memory nor torch's allocator statistics."""
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    p = pkg()
    B, H, S, D = 2, 4, 384, 64
    q, k, v, go = _case(oracle, B, H, S, D, 950)
    tq, tk, tv, tg = to_dev(q, k, v, go)
    out, lse = p.forward(tq, tk, tv, H, 0.125, True)
    grads = [torch.empty_like(tq) for _ in range(3)]
    p.backward_static_scratch(tq, tk, tv, out, tg, lse, H, 0.125, True, d_q=grads[0], d_k=grads[1], d_v=grads[2])
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    allocs_before = torch.cuda.memory_stats()["allocation.all.allocated"]
    for _ in range(3):
        p.backward_static_scratch(tq, tk, tv, out, tg, lse, H, 0.125, True, d_q=grads[0], d_k=grads[1], d_v=grads[2])
    torch.cuda.synchronize()
    assert p.sync_status() == 0
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocs_before


def test_static_scratch_limit_is_refused_before_launch():
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    p = pkg()
    L = p.lib()
    t = torch.zeros(16, device="cuda")
    ptr = t.data_ptr()
    L.df_attn_last_status()
    before = p.launch_count()
    # batch*heads*seq_len = 2 * 16 * 65537 > 2097152 rows: refused by size alone, pointers are never touched
    st = L.df_attn_backward_static_scratch(ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, 2, 16, 65537, 64, 0.125, 1,
                                           None)
    assert st == p.DF_ERR_STATIC_SCRATCH
    assert b"DF_STATIC_SCRATCH_MAX_ROWS" in L.df_attn_status_string(st)
    assert p.launch_count() == before
    assert L.df_attn_last_status() == p.DF_ERR_STATIC_SCRATCH
    assert p.sync_status() == 0
