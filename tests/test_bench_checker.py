"""The float64 sampled-row checker that bench.py applies to its multi-GPU workloads at sizes the CPU oracle cannot
reach (bench.sampled_rows_check), validated here on the CPU against the oracle at a small size: given the oracle's
own outputs it must report errors at fp32 rounding level, and given a corrupted row it must notice."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def test_sampled_rows_check_agrees_with_the_oracle(oracle):
    import torch
    import bench
    H, S, D = 3, 320, 16
    scale = 0.25
    q, k, v, go = (oracle.fill_normal((1, S, H * D), 88, st) for st in range(4))
    out, lse = oracle.forward(q, k, v, H, scale, True, f64=True)
    dq, dk, dv = oracle.backward(q, k, v, go, H, scale, True, f64=True)
    delta = oracle.delta(out, go, H)
    full = tuple(torch.from_numpy(x[0]) for x in (q, k, v, go))
    rows = torch.tensor([0, 1, 63, 64, 200, 319])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    res = bench.sampled_rows_check(torch, full, H, scale, rows, t(out[0][rows.numpy()]), t(lse[0][:, rows.numpy()]),
                                   grads=(t(dq[0][rows.numpy()]), t(dk[0][rows.numpy()]), t(dv[0][rows.numpy()]), t(lse[0]), t(delta[0])),
                                   chunk=128)
    assert res["rows"] == 6
    assert res["max_abs_err_o"] <= 1e-5 and res["max_abs_err_lse"] <= 1e-5 and res["max_rel_err_grad"] <= 1e-4, res
    bad = out[0][rows.numpy()].copy()
    bad[3, 5] += 0.01
    res_bad = bench.sampled_rows_check(torch, full, H, scale, rows, t(bad), t(lse[0][:, rows.numpy()]), chunk=128)
    assert res_bad["max_abs_err_o"] >= 9e-3
    wrong_dk = dk[0][rows.numpy()].copy() * 1.05
    res_bad = bench.sampled_rows_check(torch, full, H, scale, rows, t(out[0][rows.numpy()]), t(lse[0][:, rows.numpy()]),
                                       grads=(t(dq[0][rows.numpy()]), t(wrong_dk), t(dv[0][rows.numpy()]), t(lse[0]), t(delta[0])),
                                       chunk=128)
    assert res_bad["max_rel_err_grad"] >= 2e-2


def test_raw_step_calls_match_the_bound_prototypes():
    """bench.py's timed loops call df_attn_forward / df_attn_backward with argument tuples prepared once. On the CPU the
    tuples cannot be launched, but their arity and order can be checked against the prototypes the package binds (which
    tests/test_abi.py checks against the header): pointers first, then batch, heads, sequence, head dimension, scale,
    causal flag, stream."""
    import ctypes
    import bench
    from helpers import pkg
    p = pkg()

    class FakeTensor:
        is_cuda = True

        def __init__(self, addr):
            self.addr = addr

        def is_contiguous(self):
            return True

        def data_ptr(self):
            return self.addr

    class FakeStream:
        cuda_stream = 0x5000

    names = ("q", "k", "v", "go", "out", "lse", "delta", "dq", "dk", "dv")
    s = {n: FakeTensor(0x1000 * (i + 1)) for i, n in enumerate(names)}

    class FakeLib:
        df_attn_forward = "fwd"
        df_attn_backward = "bwd"

    class FakePkg:
        @staticmethod
        def lib():
            return FakeLib

    (f_fn, f_args), (b_fn, b_args) = bench.raw_step_calls(FakePkg, s, 8, 12, 1024, 64, 0.125, FakeStream)
    assert (f_fn, b_fn) == ("fwd", "bwd")
    for name, args in (("df_attn_forward", f_args), ("df_attn_backward", b_args)):
        restype, argtypes = p.PROTOTYPES[name]
        assert restype is ctypes.c_int and len(argtypes) == len(args), name
        assert args[-1] == 0x5000 and args[-2] == 1 and abs(args[-3] - 0.125) < 1e-12 and args[-7:-3] == (8, 12, 1024, 64), name
    assert f_args[:5] == tuple(s[n].addr for n in ("q", "k", "v", "out", "lse"))
    assert b_args[:10] == tuple(s[n].addr for n in ("q", "k", "v", "out", "go", "lse", "dq", "dk", "dv", "delta"))
