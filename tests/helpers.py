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


def sampled_backward_reference(q, k, v, go, H, scale, q_rows, k_rows, causal=True, chunk=2048, torch_device=None):
    """float64 gradients of causal attention for a SAMPLE of rows of one long sequence, without an
    S x S matrix in memory: dQ for the query rows `q_rows`, dK and dV for the key rows `k_rows`.
    q, k, v, go: [1, S, H*D] float32. Returns (dq [len(q_rows), H*D], dk, dv [len(k_rows), H*D]).

    Row statistics (logsumexp, delta = rowsum(dO o O)) are needed for every query row that sees a
    sampled key, i.e. for the whole sequence; they are computed in query chunks. With
    `torch_device` the chunked float64 products run on that torch device (the checker may use the
    GPU's float64 units: it never touches the library under test)."""
    import torch
    dev = torch.device(torch_device or "cpu")
    _, S, dm = q.shape
    D = dm // H
    tq, tk, tv, tg = (torch.from_numpy(np.ascontiguousarray(x[0])).to(dev).double().view(S, H, D).transpose(0, 1)
                      for x in (q, k, v, go))  # [H, S, D]
    lse = torch.empty((H, S), dtype=torch.float64, device=dev)
    dlt = torch.empty((H, S), dtype=torch.float64, device=dev)
    ar = torch.arange(S, device=dev)
    for c0 in range(0, S, chunk):
        c1 = min(S, c0 + chunk)
        nk = c1 if causal else S
        s = torch.einsum("hid,hjd->hij", tq[:, c0:c1], tk[:, :nk]) * scale
        if causal:
            s = s.masked_fill(ar[None, :nk] > ar[c0:c1, None], float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        o = torch.einsum("hij,hjd->hid", torch.exp(s - l[..., None]), tv[:, :nk])
        lse[:, c0:c1] = l
        dlt[:, c0:c1] = (o * tg[:, c0:c1]).sum(-1)
    q_rows = torch.as_tensor(np.asarray(q_rows), device=dev)
    k_rows = torch.as_tensor(np.asarray(k_rows), device=dev)
    # dQ rows: dS_ij = P_ij (dP_ij - delta_i), dQ_i = scale * sum_j dS_ij K_j
    s = torch.einsum("hid,hjd->hij", tq[:, q_rows], tk) * scale
    if causal:
        s = s.masked_fill(ar[None, :] > q_rows[:, None], float("-inf"))
    p = torch.exp(s - lse[:, q_rows][..., None])
    dp = torch.einsum("hid,hjd->hij", tg[:, q_rows], tv)
    ds = p * (dp - dlt[:, q_rows][..., None])
    dq = scale * torch.einsum("hij,hjd->hid", ds, tk)
    # dK, dV rows: all queries against the sampled keys, in query chunks
    dk = torch.zeros((H, len(k_rows), D), dtype=torch.float64, device=dev)
    dv = torch.zeros_like(dk)
    for c0 in range(0, S, chunk):
        c1 = min(S, c0 + chunk)
        s = torch.einsum("hid,hjd->hij", tq[:, c0:c1], tk[:, k_rows]) * scale
        if causal:
            s = s.masked_fill(k_rows[None, :] > ar[c0:c1, None], float("-inf"))
        p = torch.exp(s - lse[:, c0:c1][..., None])
        dp = torch.einsum("hid,hjd->hij", tg[:, c0:c1], tv[:, k_rows])
        ds = p * (dp - dlt[:, c0:c1][..., None])
        dv += torch.einsum("hij,hid->hjd", p, tg[:, c0:c1])
        dk += scale * torch.einsum("hij,hid->hjd", ds, tq[:, c0:c1])
    back = lambda t: t.transpose(0, 1).reshape(t.shape[1], dm).cpu().numpy()
    return back(dq), back(dk), back(dv)


def default_scale(D):
    return 1.0 / math.sqrt(D)
