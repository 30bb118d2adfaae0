"""GPU parity of the projections around the attention op (df_linear_qkv_forward, df_linear_forward), through the C ABI,
against the CPU oracle (cpu_linear restated) and the committed float64 golden vectors. Tolerance: the kernel
multiplies in TF32 like the attention op, so |out - ref| <= 2e-3 * max(1, max|ref|) for unit-variance rows and
N(0, 0.02) weights at in_features = 768 (measured error is about a tenth of that)."""
import numpy as np
import pytest

import helpers as hp
from helpers import pkg, to_dev

pytestmark = pytest.mark.gpu


def _tol(ref):
    return 2e-3 * max(1.0, float(np.abs(ref).max()))


def _case(oracle, rows, fin, fout, seed):
    x = oracle.fill_normal((rows, fin), seed, 0)
    ws = [(oracle.fill_normal((fout, fin), seed, 10 + j) * 0.02).astype(np.float32) for j in range(3)]
    bs = [(oracle.fill_normal((fout,), seed, 20 + j) * 0.02).astype(np.float32) for j in range(3)]
    r = oracle.fill_normal((rows, fout), seed, 3)
    return x, ws, bs, r


def test_linear_golden_vectors(oracle, golden):
    import torch
    torch.cuda.set_device(0)
    p = pkg()
    for name, (rows, fin, fout, seed) in zip(golden["lin_cases"], golden["lin_case_params"]):
        x = oracle.fill_normal((int(rows), int(fin)), int(seed), 0)
        w = (oracle.fill_normal((int(fout), int(fin)), int(seed), 1) * 0.02).astype(np.float32)
        b = (oracle.fill_normal((int(fout),), int(seed), 2) * 0.02).astype(np.float32)
        r = oracle.fill_normal((int(rows), int(fout)), int(seed), 3)
        tx, tw, tb, tr = to_dev(x, w, b, r)
        out = p.linear(tx, tw, tb).cpu().numpy()
        out_res = p.linear(tx, tw, tb, residual=tr).cpu().numpy()
        assert p.sync_status() == 0
        assert np.abs(out - golden[f"{name}_out"]).max() <= _tol(golden[f"{name}_out"]), name
        assert np.abs(out_res - golden[f"{name}_out_res"]).max() <= _tol(golden[f"{name}_out_res"]), name


@pytest.mark.parametrize("rows,fin,fout", [(1, 32, 256), (5, 64, 64), (127, 96, 260), (128, 768, 768), (300, 768, 768),
                                           (1000, 100, 516), (4096, 768, 768)])
def test_qkv_projection_matches_oracle(oracle, rows, fin, fout):
    """One launch for Q, K and V over ragged and tile-aligned shapes (rows not a multiple of 128, out_features not a
    multiple of 256, in_features not a multiple of 32), with and without biases; then the output projection with
    bias and residual. Guard bytes around every output stay intact."""
    import torch
    torch.cuda.set_device(0)
    p = pkg()
    x, ws, bs, r = _case(oracle, rows, fin, fout, 7000 + rows + fin)
    tx, tr = to_dev(x, r)
    tws, tbs = to_dev(*ws), to_dev(*bs)
    pad, canary = 1024, 777.0
    bufs = [torch.full((rows * fout + 2 * pad,), canary, device="cuda") for _ in range(3)]
    outs = [b[pad:pad + rows * fout].view(rows, fout) for b in bufs]
    p.linear_qkv(tx, *tws, *tbs, q=outs[0], k=outs[1], v=outs[2])
    assert p.sync_status() == 0
    for j in range(3):
        ref = oracle.linear(x, ws[j], bs[j])
        assert np.abs(outs[j].cpu().numpy() - ref).max() <= _tol(ref), (j, rows, fin, fout)
        assert bool((bufs[j][:pad] == canary).all()) and bool((bufs[j][pad + rows * fout:] == canary).all())
    q2, k2, v2 = p.linear_qkv(tx, *tws)
    for j, got in enumerate((q2, k2, v2)):
        ref = oracle.linear(x, ws[j])
        assert np.abs(got.cpu().numpy() - ref).max() <= _tol(ref), ("nobias", j)
    ref = oracle.linear(x, ws[0], bs[0], residual=r)
    got = p.linear(tx, tws[0], tbs[0], residual=tr)
    assert p.sync_status() == 0
    assert np.abs(got.cpu().numpy() - ref).max() <= _tol(ref)
    # twice the same call gives the same bits (no atomics, fixed summation order)
    again = p.linear(tx, tws[0], tbs[0], residual=tr)
    assert torch.equal(got, again)


def test_projection_feeds_attention_layout(oracle):
    """The Q, K, V written by the projection are consumed as they are by the attention entry point: [S, H*D] rows,
    head h in columns h*D..: projection + attention against oracle.linear + oracle.forward."""
    import torch
    torch.cuda.set_device(0)
    p = pkg()
    S, H, D = 384, 4, 64
    dm = H * D
    x, ws, bs, _ = _case(oracle, S, dm, dm, 4242)
    ws = [w * 3.0 for w in ws]  # scores of order one
    tx = to_dev(x)[0]
    tws, tbs = to_dev(*ws), to_dev(*bs)
    q, k, v = p.linear_qkv(tx, *tws, *tbs)
    out, lse = p.forward(q[None], k[None], v[None], H, 0.125, True)
    assert p.sync_status() == 0
    rq, rk, rv = (oracle.linear(x, w, b)[None] for w, b in zip(ws, bs))
    o_ref, lse_ref = oracle.forward(rq, rk, rv, H, 0.125, True)
    assert np.abs(out.cpu().numpy() - o_ref).max() <= 2 * hp.TOL_O_TF32
    assert np.abs(lse.cpu().numpy() - lse_ref).max() <= 2 * hp.TOL_LSE_TF32


def test_projection_rejects_what_it_cannot_run():
    import torch
    torch.cuda.set_device(0)
    p = pkg()
    L = p.lib()
    t = torch.zeros(4096, device="cuda")
    ptr = t.data_ptr()
    L.df_attn_last_status()
    # in_features not a multiple of 4: the row pitch is not 16-byte aligned
    assert L.df_linear_forward(ptr, ptr, None, None, ptr + 8192, 4, 30, 32, None) == p.DF_ERR_UNSUPPORTED
    # two of three biases
    assert L.df_linear_qkv_forward(ptr, ptr, ptr, ptr, ptr, None, ptr, ptr, ptr, ptr, 4, 32, 32, None) == p.DF_ERR_INVALID_ARG
    assert L.df_linear_forward(ptr, ptr, None, None, ptr, 0, 32, 32, None) == p.DF_OK  # no rows: nothing to do
    L.df_attn_last_status()
    assert p.sync_status() == 0


@pytest.mark.parametrize("rows,fin,fout", [(1, 4, 4), (5, 64, 64), (129, 96, 260), (300, 768, 3072), (1000, 100, 516)])
def test_projection_with_gelu_epilogue(oracle, rows, fin, fout):
    """df_linear_gelu_forward: the pre-activation equals df_linear_forward's output bit for bit (same accumulators, same
    bias add), the activated output equals df_gelu_forward of that pre-activation bit for bit (same function), both
    agree with the oracle's linear -> gelu within the projection's TF32 tolerance, guard bytes around both outputs stay
    intact, and without a pre-activation buffer the activated output is unchanged."""
    import torch
    torch.cuda.set_device(0)
    p = pkg()
    x, ws, bs, _ = _case(oracle, rows, fin, fout, 7100 + rows + fin)
    w = (ws[0] * (25.0 if fin < 32 else 1.0)).astype(np.float32)   # a few pre-activations beyond +-1 at small widths too
    tx, tw, tb = to_dev(x, w, bs[0])
    pad, canary = 1024, 777.0
    bufs = [torch.full((rows * fout + 2 * pad,), canary, device="cuda") for _ in range(2)]
    pre, act = (b[pad:pad + rows * fout].view(rows, fout) for b in bufs)
    p.linear_gelu(tx, tw, tb, pre_activation=pre, out=act)
    assert p.sync_status() == 0
    for b in bufs:
        assert float(b[:pad].min()) == canary and float(b[:pad].max()) == canary
        assert float(b[-pad:].min()) == canary and float(b[-pad:].max()) == canary
    plain = p.linear(tx, tw, tb)
    assert torch.equal(pre, plain)
    assert torch.equal(act, p.gelu(plain))
    ref_pre = oracle.linear(x, w, bs[0], f64=True)
    ref_act = oracle.gelu(ref_pre, f64=True)
    assert np.abs(pre.cpu().numpy() - ref_pre).max() <= _tol(ref_pre)
    assert np.abs(act.cpu().numpy() - ref_act).max() <= _tol(ref_pre)   # |gelu'| <= 1.13
    _, act_only = p.linear_gelu(tx, tw, tb, keep_pre_activation=False)
    assert p.sync_status() == 0
    assert torch.equal(act_only, act)
    # no bias
    pre_nb, act_nb = p.linear_gelu(tx, tw)
    assert torch.equal(pre_nb, p.linear(tx, tw)) and torch.equal(act_nb, p.gelu(pre_nb))
    # unsupported shapes are refused, nothing falls back
    if fin > 4:
        with pytest.raises(p.AttentionError):   # in_features not a multiple of 4
            p.linear_gelu(tx[:, : fin - 1].contiguous(), tw[:, : fin - 1].contiguous(), tb)
        p.lib().df_attn_last_status()
