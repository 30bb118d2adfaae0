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
