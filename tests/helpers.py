"""Shared helpers for the GPU parity tests."""
import math
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from __graft_entry__ import load_package  # noqa: E402

# Tolerances of the TF32 tensor-core path against the fp32 reference path
# (max abs error on O <= 2e-3; relative error on dQ/dK/dV <= 5e-3 of the tensor's max).
TOL_O_TF32 = 2e-3
TOL_LSE_TF32 = 2e-3
TOL_GRAD_REL_TF32 = 5e-3
# The SIMT path computes in fp32 like the reference; only summation order differs.
TOL_O_FP32 = 2e-5
TOL_GRAD_REL_FP32 = 2e-5


def pkg():
    return load_package()


def to_dev(*arrays, device="cuda"):
    import torch
    return tuple(torch.from_numpy(np.ascontiguousarray(a)).to(device) for a in arrays)


GRAD_FLOOR = 0.25


def rel_err(got, ref):
    """max|got - ref| / max(max|ref|, GRAD_FLOOR): the relative error of a gradient tensor, with an
    absolute floor so that a tensor whose true value vanishes (S = 1: dQ = dK = 0) is held to
    GRAD_FLOOR * tolerance absolute instead of dividing by zero."""
    ref = np.asarray(ref, np.float64)
    denom = max(float(np.abs(ref).max()), GRAD_FLOOR)
    return float(np.abs(np.asarray(got, np.float64) - ref).max() / denom)


def sampled_rows_reference(q, k, v, H, scale, rows, causal=True, shift=0):
    """float64 attention for a sample of query rows. q [B,Sq,H*D], k,v [B,Sk,H*D].
    Returns out [B,len(rows),H*D], lse [B,H,len(rows)]."""
    B, Sq, dm = q.shape
    Sk = k.shape[1]
    D = dm // H
    out = np.zeros((B, len(rows), dm))
    lse = np.full((B, H, len(rows)), -np.inf)
    kk = k.reshape(B, Sk, H, D).astype(np.float64)
    vv = v.reshape(B, Sk, H, D).astype(np.float64)
    for n, i in enumerate(rows):
        nk = min(Sk, i + shift + 1) if causal else Sk
        if nk <= 0:
            continue
        qi = q[:, i].reshape(B, H, D).astype(np.float64)
        s = np.einsum("bhd,bjhd->bhj", qi, kk[:, :nk]) * scale
        m = s.max(-1, keepdims=True)
        w = np.exp(s - m)
        l = w.sum(-1, keepdims=True)
        out[:, n] = np.einsum("bhj,bjhd->bhd", w / l, vv[:, :nk]).reshape(B, dm)
        lse[:, :, n] = (m + np.log(l))[..., 0]
    return out, lse


def default_scale(D):
    return 1.0 / math.sqrt(D)
