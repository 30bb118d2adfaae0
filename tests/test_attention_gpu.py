"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle and the
committed golden vectors. Bars: fp32 (SIMT) path 2e-5; TF32 tensor-core path max abs error on
O <= 2e-3 and relative error on dQ/dK/dV <= 5e-3 (of the reference tensor's max)."""
import math
import os

import numpy as np
import pytest

import helpers as hp
from helpers import pkg, rel_err, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "these tests need a GPU"
    torch.cuda.set_device(0)
    p = pkg()
    assert os.path.exists(p.LIB_PATH), "the CUDA library must be prebuilt in-tree"
    p.lib()
    yield torch
    assert p.sync_status() == 0


def _inputs(oracle, B, H, S, D, seed, Sk=None):
    q = oracle.fill_normal((B, S, H * D), seed, 0)
    k = oracle.fill_normal((B, Sk or S, H * D), seed, 1)
    v = oracle.fill_normal((B, Sk or S, H * D), seed, 2)
    go = oracle.fill_normal((B, S, H * D), seed, 3)
    return q, k, v, go


def _run_fwd_bwd(p, q, k, v, go, H, scale, causal, variant):
    prev = p.set_variant(variant)
    try:
        tq, tk, tv, tg = to_dev(q, k, v, go)
        out, lse = p.forward(tq, tk, tv, H, scale, causal)
        dq, dk, dv = p.backward(tq, tk, tv, out, tg, lse, H, scale, causal)
        assert p.sync_status() == 0
        return tuple(t.cpu().numpy() for t in (out, lse, dq, dk, dv))
    finally:
        p.set_variant(prev)


# ------------------------------------------------------------------ reference known-answer tests
def test_reference_forward_known_answer_through_legacy_api(torch_cuda, golden):
    """darkforest-cuda/src/lib.rs:2606-2628: single head, S=5, D=4, tolerance 2e-4."""
    p = pkg()
    q, k, v = (golden[f"kat_fwd_{n}"].reshape(-1) for n in ("q", "k", "v"))
    out = p.fused_attention_forward(q, k, v, 5, 4, 1.0 / math.sqrt(4.0), True)
    assert np.abs(out - golden["kat_fwd_out"].reshape(-1)).max() <= 2e-4


def test_reference_backward_known_answer_and_finite_difference(torch_cuda, golden):
    """lib.rs:2753-2829: single head, S=4, D=3; 2e-4 vs the closed form, 2e-3 vs central differences."""
    p = pkg()
    q, k, v, go = (golden[f"kat_bwd_{n}"].reshape(-1).astype(np.float32) for n in ("q", "k", "v", "do"))
    scale = 1.0 / math.sqrt(3.0)
    grads = p.attention_backward(q, k, v, go, 4, 3, scale, True)
    for g, n in zip(grads, ("dq", "dk", "dv")):
        assert np.abs(g - golden[f"kat_bwd_{n}"].reshape(-1)).max() <= 2e-4, n

    def objective(q_, k_, v_):
        return float((p.fused_attention_forward(q_, k_, v_, 4, 3, scale, True).astype(np.float64) * go).sum())

    delta = 1e-3
    base = [q, k, v]
    for which, analytical in enumerate(grads):
        for index in range(analytical.size):
            plus = [a.copy() for a in base]
            minus = [a.copy() for a in base]
            plus[which][index] += delta
            minus[which][index] -= delta
            numerical = (objective(*plus) - objective(*minus)) / (2 * delta)
            assert abs(analytical[index] - numerical) <= 2e-3


# ------------------------------------------------------------------ golden vectors
@pytest.mark.parametrize("name", ["mh_small", "mh_noncausal", "mh_d128", "mh_ragged", "mh_cfg1"])
@pytest.mark.parametrize("variant", ["simt", "auto"])
def test_golden_multihead(torch_cuda, oracle, golden, name, variant):
    p = pkg()
    idx = list(golden["cases"]).index(name)
    B, H, S, D, causal, seed = (int(x) for x in golden["case_params"][idx])
    q, k, v, go = _inputs(oracle, B, H, S, D, seed)
    rows = golden[f"{name}_rows"]
    var = p.VARIANT_SIMT if variant == "simt" else p.VARIANT_AUTO
    out, lse, dq, dk, dv = _run_fwd_bwd(p, q, k, v, go, H, hp.default_scale(D), bool(causal), var)
    tensor = variant == "auto" and D == 64
    tol_o = hp.TOL_O_TF32 if tensor else hp.TOL_O_FP32
    tol_g = hp.TOL_GRAD_REL_TF32 if tensor else hp.TOL_GRAD_REL_FP32
    assert np.abs(out[:, rows] - golden[f"{name}_out"]).max() <= tol_o
    assert np.abs(lse[:, :, rows] - golden[f"{name}_lse"]).max() <= tol_o * 4
    for g, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert rel_err(g[:, rows], golden[f"{name}_{n}"]) <= tol_g, n


# ------------------------------------------------------------------ shape sweep against the oracle
SWEEP = [(1, 1, S, D) for S in (1, 2, 3, 5, 31, 33, 127, 129, 257) for D in (3, 4, 32, 64, 128)] + \
        [(2, 3, 65, 64), (1, 12, 128, 64), (2, 2, 255, 64), (1, 2, 384, 64), (1, 3, 200, 96)]


@pytest.mark.parametrize("causal", [True, False])
def test_shape_sweep_simt(torch_cuda, oracle, causal):
    p = pkg()
    for B, H, S, D in SWEEP:
        q, k, v, go = _inputs(oracle, B, H, S, D, 1000 + S * 131 + D)
        scale = hp.default_scale(D)
        out, lse, dq, dk, dv = _run_fwd_bwd(p, q, k, v, go, H, scale, causal, p.VARIANT_SIMT)
        o_ref, lse_ref = oracle.forward(q, k, v, H, scale, causal)
        g_ref = oracle.backward(q, k, v, go, H, scale, causal)
        tag = (B, H, S, D, causal)
        assert np.abs(out - o_ref).max() <= hp.TOL_O_FP32, tag
        assert np.abs(lse - lse_ref).max() <= 1e-4, tag
        for g, r in zip((dq, dk, dv), g_ref):
            assert np.abs(g - r).max() <= 1e-4 * max(1.0, np.abs(r).max()), tag


@pytest.mark.parametrize("persist", [0, 2])
@pytest.mark.parametrize("causal", [True, False])
def test_shape_sweep_tensor_forward(torch_cuda, oracle, causal, persist):
    """tcgen05 forward at D=64 over ragged and tile-aligned S, several batch/head counts, through both
    whole-sequence kernels: one CTA per pair of query tiles (0) and the persistent one (2)."""
    p = pkg()
    prev_opt = p.set_option(p.OPT_FWD_PERSIST, persist)
    prev = p.set_variant(p.VARIANT_TENSOR)
    try:
        for B, H, S in [(1, 1, 1), (1, 2, 5), (1, 1, 127), (1, 1, 128), (1, 2, 129), (2, 3, 257), (1, 12, 128),
                        (2, 2, 384), (1, 1, 1000), (3, 5, 640), (1, 40, 1300)]:
            q, k, v, _ = _inputs(oracle, B, H, S, 64, 2000 + S)
            tq, tk, tv = to_dev(q, k, v)
            out, lse = p.forward(tq, tk, tv, H, 0.125, causal)
            assert p.sync_status() == 0
            o_ref, lse_ref = oracle.forward(q, k, v, H, 0.125, causal)
            tag = (B, H, S, causal)
            assert np.abs(out.cpu().numpy() - o_ref).max() <= hp.TOL_O_TF32, tag
            assert np.abs(lse.cpu().numpy() - lse_ref).max() <= hp.TOL_LSE_TF32, tag
    finally:
        p.set_variant(prev)
        p.set_option(p.OPT_FWD_PERSIST, prev_opt)


@pytest.mark.parametrize("causal", [True, False])
def test_shape_sweep_tensor_backward(torch_cuda, oracle, causal):
    """tcgen05 dK/dV and dQ kernels at D=64 over ragged and tile-aligned S."""
    p = pkg()
    for B, H, S in [(1, 1, 1), (1, 2, 5), (1, 1, 127), (1, 1, 128), (1, 2, 129), (2, 3, 257), (1, 12, 128),
                    (2, 2, 384), (1, 2, 1000), (1, 40, 1300)]:
        q, k, v, go = _inputs(oracle, B, H, S, 64, 3000 + S)
        out, lse, dq, dk, dv = _run_fwd_bwd(p, q, k, v, go, H, 0.125, causal, p.VARIANT_TENSOR)
        g_ref = oracle.backward(q, k, v, go, H, 0.125, causal)
        for g, r, n in zip((dq, dk, dv), g_ref, ("dq", "dk", "dv")):
            assert rel_err(g, r) <= hp.TOL_GRAD_REL_TF32, (B, H, S, causal, n)


def test_tensor_path_is_taken_for_the_benchmark_shapes(torch_cuda):
    p = pkg()
    t = torch_cuda.zeros((1024, 768), device="cuda")
    assert p.lib().df_attn_forward_uses_tensor_cores(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                                     12, 1024, 1024, 64) == 1
    assert p.lib().df_attn_forward_uses_tensor_cores(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                                     8, 1024, 1024, 96) == 0


# ------------------------------------------------------------------ legacy multi-head API (drop-in)
def test_legacy_mha_api_cfg1(torch_cuda, oracle):
    """B=1,H=12,S=128,D=64 through AttentionContext.forward_device_into / backward_device_into."""
    p = pkg()
    H, S, D = 12, 128, 64
    q, k, v, go = _inputs(oracle, 1, H, S, D, 0xDF01)
    ctx = p.AttentionContext(H, S, D)
    tq, tk, tv, tg = (t[0].contiguous() for t in to_dev(q, k, v, go))
    out = ctx.forward_device(tq, tk, tv, 0.125, True)
    dq, dk, dv = ctx.backward_device(tq, tk, tv, tg, 0.125, True)
    assert p.sync_status() == 0
    o_ref, _ = oracle.forward(q, k, v, H, 0.125, True)
    g_ref = oracle.backward(q, k, v, go, H, 0.125, True)
    assert np.abs(out.cpu().numpy() - o_ref[0]).max() <= hp.TOL_O_TF32
    for g, r in zip((dq, dk, dv), g_ref):
        assert rel_err(g.cpu().numpy(), r[0]) <= hp.TOL_GRAD_REL_TF32


def test_legacy_backward_tiny_scratch_and_single_key(torch_cuda, oracle):
    """S so small that the caller's H*2*S*S scratch cannot hold O; and S = 1."""
    p = pkg()
    for H, S, D in [(2, 3, 64), (1, 2, 128), (3, 1, 64), (1, 1, 7)]:
        q, k, v, go = _inputs(oracle, 1, H, S, D, 31 + S + D)
        ctx = p.AttentionContext(H, S, D)
        tq, tk, tv, tg = (t[0].contiguous() for t in to_dev(q, k, v, go))
        dq, dk, dv = ctx.backward_device(tq, tk, tv, tg, 0.3, True)
        assert p.sync_status() == 0
        # D = 64 runs on the TF32 tensor-core kernels, the other head sizes on the fp32 SIMT kernels
        tol = hp.TOL_GRAD_REL_TF32 if D == 64 else hp.TOL_GRAD_REL_FP32
        for g, r in zip((dq, dk, dv), oracle.backward(q, k, v, go, H, 0.3, True)):
            assert rel_err(g.cpu().numpy(), r[0]) <= tol, (H, S, D)


# ------------------------------------------------------------------ the oracle against the real reference
def test_oracle_matches_reference_cuda_kernels(torch_cuda, oracle):
    """Pins the CPU restatement against the reference's own CUDA kernels
    (darkforest-cuda/kernels/attention_fused.cu compiled unmodified for sm_100a)."""
    from oracle.attn_oracle import REFERENCE_SO, ReferenceKernels
    if not os.path.exists(REFERENCE_SO):
        pytest.skip("oracle/_ref was not built (reference source tree absent at build time)")
    ref = ReferenceKernels()
    for H, S, D in [(12, 128, 64), (3, 200, 64), (2, 77, 32)]:
        q, k, v, go = _inputs(oracle, 1, H, S, D, 500 + S)
        tq, tk, tv, tg = (t[0].contiguous() for t in to_dev(q, k, v, go))
        scale = hp.default_scale(D)
        out = ref.mha_forward(tq, tk, tv, H, scale, True).cpu().numpy()
        dq, dk, dv = (t.cpu().numpy() for t in ref.mha_backward(tq, tk, tv, tg, H, scale, True))
        o_ref, _ = oracle.forward(q, k, v, H, scale, True)
        g_ref = oracle.backward(q, k, v, go, H, scale, True)
        assert np.abs(out - o_ref[0]).max() <= 2e-5, (H, S, D)
        for g, r in zip((dq, dk, dv), g_ref):
            assert np.abs(g - r[0]).max() <= 2e-4 * max(1.0, np.abs(r).max()), (H, S, D)


# ------------------------------------------------------------------ blocks, merge, helpers
@pytest.mark.parametrize("variant", ["simt", "auto"])
def test_forward_block_with_causal_shift_and_merge(torch_cuda, oracle, variant):
    """Two key blocks of a causal problem computed separately and merged equal the whole."""
    p = pkg()
    prev = p.set_variant(p.VARIANT_SIMT if variant == "simt" else p.VARIANT_AUTO)
    try:
        B, H, S, D = 1, 2, 320, 64
        q, k, v, go = _inputs(oracle, B, H, S, D, 42)
        half = 192
        tq, tk, tv = to_dev(q, k, v)
        # queries of the second part [half, S) against keys [0, half) and [half, S)
        tq2 = tq[:, half:].contiguous()
        o_a, l_a = p.forward(tq2, tk[:, :half].contiguous(), tv[:, :half].contiguous(), H, 0.125, True,
                             causal_shift=half)
        o_b, l_b = p.forward(tq2, tk[:, half:].contiguous(), tv[:, half:].contiguous(), H, 0.125, True,
                             causal_shift=0)
        p.merge_partials(o_a, l_a, o_b, l_b, H)
        # a block that lies entirely above the diagonal: nothing visible
        o_c, l_c = p.forward(tq[:, :64].contiguous(), tk[:, 128:].contiguous(), tv[:, 128:].contiguous(), H, 0.125,
                             True, causal_shift=-128)
        assert p.sync_status() == 0
        o_ref, lse_ref = oracle.forward(q, k, v, H, 0.125, True)
        tol = hp.TOL_O_TF32 if variant == "auto" else hp.TOL_O_FP32
        assert np.abs(o_a.cpu().numpy() - o_ref[:, half:]).max() <= tol
        assert np.abs(l_a.cpu().numpy() - lse_ref[:, :, half:]).max() <= tol
        assert float(o_c.abs().max()) == 0.0 and bool(torch_cuda.isinf(l_c).all())
    finally:
        p.set_variant(prev)


@pytest.mark.parametrize("variant,D,S,half", [("simt", 32, 96, 64), ("tensor", 64, 416, 256), ("tensor", 64, 300, 100)])
def test_backward_block_sums_to_full_backward(torch_cuda, oracle, variant, D, S, half):
    p = pkg()
    prev = p.set_variant(p.VARIANT_SIMT if variant == "simt" else p.VARIANT_TENSOR)
    try:
        B, H = 1, 2
        q, k, v, go = _inputs(oracle, B, H, S, D, 43)
        scale = hp.default_scale(D)
        tq, tk, tv, tg = to_dev(q, k, v, go)
        out, lse = p.forward(tq, tk, tv, H, scale, True)
        dlt = p.delta(out, tg, H)
        dq = torch_cuda.zeros_like(tq)
        dk = torch_cuda.zeros_like(tk)
        dv = torch_cuda.zeros_like(tv)
        for (qs, qe) in ((0, half), (half, S)):
            for (ks, ke) in ((0, half), (half, S)):
                if ks > qe - 1:
                    continue
                g = p.backward_block(tq[:, qs:qe].contiguous(), tk[:, ks:ke].contiguous(), tv[:, ks:ke].contiguous(),
                                     tg[:, qs:qe].contiguous(), lse[:, :, qs:qe].contiguous(),
                                     dlt[:, :, qs:qe].contiguous(), H, scale, True, causal_shift=qs - ks)
                dq[:, qs:qe] += g[0]
                dk[:, ks:ke] += g[1]
                dv[:, ks:ke] += g[2]
        assert p.sync_status() == 0
        for g, r in zip((dq, dk, dv), oracle.backward(q, k, v, go, H, scale, True)):
            assert rel_err(g.cpu().numpy(), r) <= (1e-4 if variant == "simt" else hp.TOL_GRAD_REL_TF32)
    finally:
        p.set_variant(prev)


def test_delta_prepass_and_accumulate(torch_cuda, oracle):
    p = pkg()
    for B, H, S, D in [(2, 12, 100, 64), (1, 3, 33, 128), (1, 2, 40, 24), (1, 5, 64, 8)]:
        o = oracle.fill_normal((B, S, H * D), 7, 0)
        g = oracle.fill_normal((B, S, H * D), 7, 1)
        to, tg = to_dev(o, g)
        d = p.delta(to, tg, H).cpu().numpy()
        assert np.abs(d - oracle.delta(o, g, H)).max() <= 1e-4, (B, H, S, D)
    a = torch_cuda.ones(1000, device="cuda")
    b = torch_cuda.full((1000,), 2.0, device="cuda")
    p.accumulate(a, b)
    assert float(a.sum()) == 3000.0


def test_outputs_are_overwritten_and_guard_bytes_intact(torch_cuda, oracle):
    """O/dQ/dK/dV are overwritten (never accumulated) and nothing is written outside them."""
    p = pkg()
    B, H, S, D = 1, 2, 130, 64
    n = B * S * H * D
    q, k, v, go = _inputs(oracle, B, H, S, D, 99)
    tq, tk, tv, tg = to_dev(q, k, v, go)
    pad = 4096
    canary = 12345.0
    for variant in (p.VARIANT_SIMT, p.VARIANT_AUTO):
        prev = p.set_variant(variant)
        try:
            bufs = [torch_cuda.full((n + 2 * pad,), canary, device="cuda") for _ in range(4)]
            views = [b[pad:pad + n].view(B, S, H * D) for b in bufs]
            lse = torch_cuda.empty((B, H, S), device="cuda")
            p.forward(tq, tk, tv, H, 0.125, True, out=views[0], lse=lse)
            p.backward(tq, tk, tv, views[0], tg, lse, H, 0.125, True, d_q=views[1], d_k=views[2], d_v=views[3])
            assert p.sync_status() == 0
            for b in bufs:
                assert bool((b[:pad] == canary).all()) and bool((b[pad + n:] == canary).all())
                assert not bool((b[pad:pad + n] == canary).any())
                assert bool(torch_cuda.isfinite(b).all())
        finally:
            p.set_variant(prev)


def test_results_are_bit_reproducible(torch_cuda, oracle):
    p = pkg()
    B, H, S, D = 1, 4, 300, 64
    q, k, v, go = _inputs(oracle, B, H, S, D, 5)
    a = _run_fwd_bwd(p, q, k, v, go, H, 0.125, True, p.VARIANT_AUTO)
    b = _run_fwd_bwd(p, q, k, v, go, H, 0.125, True, p.VARIANT_AUTO)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_unaligned_slices_fall_back_to_the_generic_kernels(torch_cuda, oracle):
    """Callers may pass offset pointers (DeviceTensor::as_ptr_offset, lib.rs:528-534)."""
    p = pkg()
    B, H, S, D = 1, 2, 64, 64
    q, k, v, go = _inputs(oracle, B, H, S, D, 11)
    n = B * S * H * D
    raw = [torch_cuda.empty(n + 1, device="cuda") for _ in range(3)]
    views = []
    for r, a in zip(raw, (q, k, v)):
        r[1:].copy_(torch_cuda.from_numpy(a.reshape(-1)))
        views.append(r[1:].view(B, S, H * D))
    assert views[0].data_ptr() % 16 == 4
    out, lse = p.forward(*views, H, 0.125, True)
    assert p.sync_status() == 0
    o_ref, _ = oracle.forward(q, k, v, H, 0.125, True)
    assert np.abs(out.cpu().numpy() - o_ref).max() <= hp.TOL_O_FP32


# ------------------------------------------------------------------ benchmark-size properties
def test_long_sequence_forward_row_sample(torch_cuda, oracle):
    """S = 8192, H = 12, D = 64 (the sweep's first point): sampled rows against float64, through the kernel the
    launcher picks at this length (one CTA per pair of query tiles) and through the persistent kernel with its
    host-computed work lists (option value 2)."""
    p = pkg()
    B, H, S, D = 1, 12, 8192, 64
    q, k, v, _ = _inputs(oracle, B, H, S, D, 0xDF03)
    tq, tk, tv = to_dev(q, k, v)
    rng = np.random.default_rng(0)
    rows = np.unique(np.r_[0:64, S - 64:S, rng.integers(0, S, 128)])
    o_ref, lse_ref = hp.sampled_rows_reference(q, k, v, H, 0.125, rows)
    v2 = oracle.fill_normal((B, S, H * D), 0xDF03, 9)
    tv2, = to_dev(v2)
    for persist in (1, 2):
        prev = p.set_option(p.OPT_FWD_PERSIST, persist)
        try:
            out, lse = p.forward(tq, tk, tv, H, 0.125, True)
            assert p.sync_status() == 0
            assert np.abs(out.cpu().numpy()[:, rows] - o_ref).max() <= hp.TOL_O_TF32, persist
            assert np.abs(lse.cpu().numpy()[:, :, rows] - lse_ref).max() <= hp.TOL_LSE_TF32, persist
            # linearity in V: O(V1 + V2) = O(V1) + O(V2) for fixed Q, K (size-independent property)
            out2, _ = p.forward(tq, tk, tv2, H, 0.125, True)
            out12, _ = p.forward(tq, tk, tv + tv2, H, 0.125, True)
            assert float((out12 - out - out2).abs().max()) <= 3 * hp.TOL_O_TF32, persist
        finally:
            p.set_option(p.OPT_FWD_PERSIST, prev)


def test_benchmark_configuration_full_parity(torch_cuda, oracle):
    """The configuration the headline number is quoted on, exactly: B=8, H=12, S=1024, D=64, causal, seed
    0xDF02, through df_attn_forward + df_attn_backward; every element of O, lse, dQ, dK, dV against the oracle."""
    p = pkg()
    B, H, S, D = 8, 12, 1024, 64
    q, k, v, go = _inputs(oracle, B, H, S, D, 0xDF02)
    out, lse, dq, dk, dv = _run_fwd_bwd(p, q, k, v, go, H, 0.125, True, p.VARIANT_TENSOR)
    o_ref, lse_ref = oracle.forward(q, k, v, H, 0.125, True)
    g_ref = oracle.backward(q, k, v, go, H, 0.125, True)
    assert np.abs(out - o_ref).max() <= hp.TOL_O_TF32
    assert np.abs(lse - lse_ref).max() <= hp.TOL_LSE_TF32
    for g, r, n in zip((dq, dk, dv), g_ref, ("dq", "dk", "dv")):
        assert rel_err(g, r) <= hp.TOL_GRAD_REL_TF32, n
    # the same call timed per kernel returns the same gradients
    tq, tk, tv, tg = to_dev(q, k, v, go)
    to, tl = to_dev(out, lse)
    pq, pk, pv, ms_dq, ms_dkdv = p.backward_profile(tq, tk, tv, to, tg, tl, H, 0.125, True)
    assert ms_dq > 0.0 and ms_dkdv > 0.0
    for a, b in zip((pq, pk, pv), (dq, dk, dv)):
        assert np.array_equal(a.cpu().numpy(), b)


@pytest.mark.parametrize("S", [16384, 32768])
def test_long_sequence_forward_backward_row_samples(torch_cuda, oracle, S):
    """The kernels that only long sequences reach, against float64 on sampled rows: S = 16384 takes the
    persistent forward with explicit work lists, S = 32768 the one-CTA-per-pair forward; both take the
    persistent backward kernels over 128 / 256 tiles per head. Forward rows, dQ rows and dK/dV rows are
    sampled at both ends of the sequence (the heaviest and the lightest tiles) and at random in between."""
    p = pkg()
    B, H, D = 1, 12, 64
    q, k, v, go = _inputs(oracle, B, H, S, D, 0xDF03 + S)
    tq, tk, tv, tg = to_dev(q, k, v, go)
    out, lse = p.forward(tq, tk, tv, H, 0.125, True)
    dq, dk, dv = p.backward(tq, tk, tv, out, tg, lse, H, 0.125, True)
    assert p.sync_status() == 0
    rng = np.random.default_rng(S)
    rows = np.unique(np.r_[0:32, S - 32:S, rng.integers(0, S, 96)])
    o_ref, lse_ref = hp.sampled_rows_reference(q, k, v, H, 0.125, rows)
    assert np.abs(out.cpu().numpy()[:, rows] - o_ref).max() <= hp.TOL_O_TF32
    assert np.abs(lse.cpu().numpy()[:, :, rows] - lse_ref).max() <= hp.TOL_LSE_TF32
    q_rows = np.unique(np.r_[0:16, S - 16:S, rng.integers(0, S, 96)])
    k_rows = np.unique(np.r_[0:8, S - 8:S, rng.integers(0, S, 48)])
    dq_ref, dk_ref, dv_ref = hp.sampled_backward_reference(q, k, v, go, H, 0.125, q_rows, k_rows, chunk=1024,
                                                           torch_device="cuda")
    # relative to the largest entry of the sampled reference rows (a lower bound of the tensor's maximum)
    assert rel_err(dq.cpu().numpy()[0, q_rows], dq_ref) <= hp.TOL_GRAD_REL_TF32
    assert rel_err(dk.cpu().numpy()[0, k_rows], dk_ref) <= hp.TOL_GRAD_REL_TF32
    assert rel_err(dv.cpu().numpy()[0, k_rows], dv_ref) <= hp.TOL_GRAD_REL_TF32


def test_block_backward_from_two_host_threads(torch_cuda, oracle):
    """Two host threads call df_attn_backward_block on the same GPU, each on its own stream, many times
    in a row; every result equals the serial one bit for bit (each thread forks to its own side stream
    and records its own events)."""
    import threading
    torch = torch_cuda
    p = pkg()
    H, S, D = 4, 640, 64
    cases = []
    for seed in (91, 92):
        q, k, v, go = _inputs(oracle, 1, H, S, D, seed)
        tq, tk, tv, tg = to_dev(q, k, v, go)
        out, lse = p.forward(tq, tk, tv, H, 0.125, True)
        dlt = p.delta(out, tg, H)
        ref = tuple(t.clone() for t in p.backward_block(tq, tk, tv, tg, lse, dlt, H, 0.125, True))
        cases.append((tq, tk, tv, tg, lse, dlt, ref))
    torch.cuda.synchronize()
    errors = []

    def worker(case):
        try:
            torch.cuda.set_device(0)
            tq, tk, tv, tg, lse, dlt, ref = case
            st = torch.cuda.Stream()
            p.init()
            for _ in range(40):
                with torch.cuda.stream(st):
                    got = p.backward_block(tq, tk, tv, tg, lse, dlt, H, 0.125, True, stream=st)
                st.synchronize()
                for a, b in zip(got, ref):
                    if not torch.equal(a, b):
                        errors.append("mismatch")
                        return
        except Exception as exc:  # surfaced below: an exception in a thread would otherwise be lost
            errors.append(repr(exc))

    threads = [threading.Thread(target=worker, args=(c,)) for c in cases]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert p.sync_status() == 0


# ------------------------------------------------------------------ ring driver on the CUDA backend
@pytest.mark.parametrize("B,S", [(8, 1024), (1, 32768)])
def test_full_size_gradient_identities(torch_cuda, B, S):
    """Benchmark-size checks that need no oracle (H = 12, D = 64; the step shape and a long sequence that
    takes the non-persistent forward): O is linear in V, so sum(dV o V) = sum(dO o O) = sum(delta); the
    scores depend on Q and K only through their products, so sum(dQ o Q) = sum(dK o K); and lse, delta
    come back finite. Sums are taken in float64; the bound is three times the TF32 gradient tolerance times the
    scale of a sum of independent per-term errors, which a gradient that is off by a few per cent exceeds."""
    torch = torch_cuda
    p = pkg()
    H, D = 12, 64
    g = torch.Generator(device="cuda")
    g.manual_seed(0xDF02 + S)
    q, k, v, go = (torch.randn((B, S, H * D), device="cuda", generator=g) for _ in range(4))
    out, lse = p.forward(q, k, v, H, 0.125, True)
    delta = torch.empty((B, H, S), device="cuda")
    dq, dk, dv = p.backward(q, k, v, out, go, lse, H, 0.125, True, delta_buf=delta)
    assert p.sync_status() == 0
    assert bool(torch.isfinite(lse).all()) and bool(torch.isfinite(delta).all())

    def dot(a, b):
        return float((a.double() * b.double()).sum())

    def spread(a, b):
        """Scale of a sum of independent per-term errors: sqrt(sum((a o b)^2))."""
        return float((a.double() * b.double()).pow(2).sum().sqrt())

    bound = 3.0 * hp.TOL_GRAD_REL_TF32
    s_vo, s_go, s_dl = dot(dv, v), dot(go, out), float(delta.double().sum())
    assert abs(s_vo - s_go) <= bound * max(spread(go, out), spread(dv, v)), (s_vo, s_go)
    assert abs(s_dl - s_go) <= bound * spread(go, out), (s_dl, s_go)
    s_q, s_k = dot(dq, q), dot(dk, k)
    assert abs(s_q - s_k) <= bound * max(spread(dq, q), spread(dk, k)), (s_q, s_k)


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_ring_driver_with_cuda_backend_single_rank(torch_cuda, oracle, layout):
    """world_size 1: the zigzag layout still splits the sequence into two chunks, so the block
    forward/backward entry points, the logsumexp merge and the accumulation all run on the GPU."""
    import importlib
    import torch.distributed as dist
    p = pkg()
    ring = importlib.import_module("dark_forest_b200.ring")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29655")
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        H, S, D = 3, 512, 64
        scale = 0.125
        q, k, v, go = _inputs(oracle, 1, H, S, D, 77)
        tq, tk, tv, tg = to_dev(q, k, v, go)
        ra = ring.RingAttention(ring.CudaBackend(p, H, scale), S, H, D, "cuda", causal=True, layout=layout)
        out, lse = torch_cuda.empty_like(tq), torch_cuda.empty((1, H, S), device="cuda")
        ra.forward(tq, tk, tv, out, lse)
        dq, dk, dv = (torch_cuda.empty_like(tq) for _ in range(3))
        ra.backward(tq, tk, tv, out, tg, lse, dq, dk, dv)
        assert p.sync_status() == 0
        o_ref, lse_ref = oracle.forward(q, k, v, H, scale, True)
        assert np.abs(out.cpu().numpy() - o_ref).max() <= hp.TOL_O_TF32
        assert np.abs(lse.cpu().numpy() - lse_ref).max() <= hp.TOL_LSE_TF32
        for g, r in zip((dq, dk, dv), oracle.backward(q, k, v, go, H, scale, True)):
            assert rel_err(g.cpu().numpy(), r) <= hp.TOL_GRAD_REL_TF32
    finally:
        if created:
            dist.destroy_process_group()


# ------------------------------------------------------------------ bf16 variant
TOL_O_BF16 = 2e-2   # bf16 output (8 mantissa bits) and bf16 P against the float64 result on the same bf16 inputs


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [True, False])
def test_bf16_forward(torch_cuda, oracle, D, causal):
    """bf16 in / bf16 out forward (kind::f16 MMA) against the oracle evaluated on the bf16-rounded inputs."""
    p = pkg()
    for B, H, S in [(1, 2, 5), (1, 1, 128), (2, 3, 257), (1, 4, 640), (1, 2, 1000)]:
        q, k, v, _ = _inputs(oracle, B, H, S, D, 4000 + S + D)
        qr, kr, vr = (oracle.round_bf16(x)[0] for x in (q, k, v))
        tq, tk, tv = (t.to(torch_cuda.bfloat16) for t in to_dev(qr, kr, vr))
        scale = hp.default_scale(D)
        out, lse = p.forward_bf16(tq, tk, tv, H, scale, causal)
        assert p.sync_status() == 0
        o_ref, lse_ref = oracle.forward(qr, kr, vr, H, scale, causal, f64=True)
        tag = (B, H, S, D, causal)
        assert np.abs(out.float().cpu().numpy() - o_ref).max() <= TOL_O_BF16, tag
        assert np.abs(lse.cpu().numpy() - lse_ref).max() <= 2e-3, tag


def test_bf16_unsupported_head_size_is_reported(torch_cuda):
    p = pkg()
    t = torch_cuda.zeros((1, 64, 2 * 96), device="cuda", dtype=torch_cuda.bfloat16)
    with pytest.raises(p.AttentionError):
        p.forward_bf16(t, t, t, 2, 0.1, True)
    assert p.lib().df_attn_last_status() == p.DF_ERR_UNSUPPORTED


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [True, False])
def test_bf16_backward(torch_cuda, oracle, D, causal):
    """bf16 gradients against the float64 oracle on the bf16-rounded inputs; 2e-2 of the tensor's max
    (bf16 P, dS and outputs carry 8 mantissa bits)."""
    p = pkg()
    for B, H, S in [(1, 2, 5), (1, 1, 128), (2, 3, 257), (1, 2, 640), (1, 2, 1000)]:
        q, k, v, go = _inputs(oracle, B, H, S, D, 5000 + S + D)
        qr, kr, vr, gr = (oracle.round_bf16(x)[0] for x in (q, k, v, go))
        tq, tk, tv, tg = (t.to(torch_cuda.bfloat16) for t in to_dev(qr, kr, vr, gr))
        scale = hp.default_scale(D)
        out, lse = p.forward_bf16(tq, tk, tv, H, scale, causal)
        dq, dk, dv = p.backward_bf16(tq, tk, tv, out, tg, lse, H, scale, causal)
        assert p.sync_status() == 0
        g_ref = oracle.backward(qr, kr, vr, gr, H, scale, causal, f64=True)
        for g, r, n in zip((dq, dk, dv), g_ref, ("dq", "dk", "dv")):
            assert rel_err(g.float().cpu().numpy(), r) <= 2e-2, (B, H, S, D, causal, n)


# ------------------------------------------------------------------ the op inside a GPT-2 step (caller side)
def test_gpt2_step_loss_parity_with_sdpa_twin(torch_cuda):
    """End-to-end check in the spirit of the reference's scripts/verify_loss_parity.py:97-158
    (vocab 500, d_model 128, 4 heads of... here 2 heads of 64, 2 layers, S=64): the loss of a small GPT-2 that
    calls this library's attention equals the loss of the same weights with torch SDPA to < 1e-3; the initial
    loss sits at ln(vocab); a few AdamW steps on a fixed batch reduce it."""
    import importlib
    import torch.nn.functional as F
    torch = torch_cuda
    p = pkg()
    step = importlib.import_module("dark_forest_b200.gpt2_step")
    model, opt, timers = step.build(p, n_layers=2, d_model=128, n_heads=2, d_ff=512, vocab=500, max_pos=64, seed=42)
    g = torch.Generator(device="cuda")
    g.manual_seed(42)
    idx = torch.randint(0, 500, (2, 64), device="cuda", generator=g)
    tgt = torch.randint(0, 500, (2, 64), device="cuda", generator=g)
    with torch.no_grad():
        loss_ours = float(model(idx, tgt))
        # twin: same weights, attention by torch SDPA in fp32
        def twin_forward(x):
            B, S = x.shape
            h = model.tok(x) + model.pos(torch.arange(S, device=x.device))[None]
            for blk in model.blocks:
                y = blk.ln1(h)
                q, k, v = (w(y).view(B, S, 2, 64).transpose(1, 2) for w in (blk.wq, blk.wk, blk.wv))
                a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, 128)
                h = h + blk.wo(a)
                h = h + blk.w2(F.gelu(blk.w1(blk.ln2(h)), approximate="tanh"))
            logits = model.ln_f(h).reshape(B * S, 128) @ model.tok.weight.t()
            return float(F.cross_entropy(logits, tgt.reshape(-1)))
        torch.backends.cuda.matmul.allow_tf32 = False
        loss_twin = twin_forward(idx)
        torch.backends.cuda.matmul.allow_tf32 = True
    assert abs(loss_ours - loss_twin) < 1e-3, (loss_ours, loss_twin)
    assert abs(loss_ours - math.log(500)) < 0.1
    losses = []
    for _ in range(8):
        loss = model(idx, tgt)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert p.sync_status() == 0
    assert losses[-1] < losses[0] - 0.05, losses
    # one attention call per layer: 1 evaluation + 8 training forwards, 8 backwards
    assert len(timers["fwd"]) == 2 * 9 and len(timers["bwd"]) == 2 * 8


# ------------------------------------------------------------------ failure path: a wait that runs out
def test_bounded_wait_expiry_is_reported_and_the_context_survives(torch_cuda, oracle):
    """No GPU fault is provoked: a kernel waits (bounded, 30 ms) on a barrier nothing signals, gives up, exits
    normally and raises the status word; the host reads DF_ERR_DEVICE_TIMEOUT once, and ordinary calls keep working."""
    p = pkg()
    L = p.lib()
    assert p.sync_status() == 0
    assert L.df_attn_selftest_wait_expiry(30, None) == 0
    assert p.sync_status() == p.DF_ERR_DEVICE_TIMEOUT
    assert p.sync_status() == 0                       # the status is reported once, then cleared
    assert L.df_attn_selftest_wait_expiry(0, None) == p.DF_ERR_INVALID_ARG
    L.df_attn_last_status()
    q, k, v, _ = _inputs(oracle, 1, 2, 256, 64, 3)
    tq, tk, tv = to_dev(q, k, v)
    out, _ = p.forward(tq, tk, tv, 2, 0.125, True)
    assert p.sync_status() == 0
    o_ref, _ = oracle.forward(q, k, v, 2, 0.125, True)
    assert np.abs(out.cpu().numpy() - o_ref).max() <= hp.TOL_O_TF32


def test_ring_driver_bf16_backend_single_rank(torch_cuda, oracle):
    """bf16 ring (D = 128): bf16 operands, fp32 partial results merged over the zigzag blocks, one final rounding."""
    import importlib
    import torch.distributed as dist
    p = pkg()
    ring = importlib.import_module("dark_forest_b200.ring")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29656")
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        H, S, D = 2, 768, 128
        scale = hp.default_scale(D)
        q, k, v, go = _inputs(oracle, 1, H, S, D, 78)
        qr, kr, vr, gr = (oracle.round_bf16(x)[0] for x in (q, k, v, go))
        bf = torch_cuda.bfloat16
        tq, tk, tv, tg = (t.to(bf) for t in to_dev(qr, kr, vr, gr))
        ra = ring.RingAttention(ring.CudaBackendBf16(p, H, scale), S, H, D, "cuda", causal=True, layout="zigzag")
        out, lse = torch_cuda.empty_like(tq), torch_cuda.empty((1, H, S), device="cuda")
        ra.forward(tq, tk, tv, out, lse)
        dq, dk, dv = (torch_cuda.empty_like(tq) for _ in range(3))
        ra.backward(tq, tk, tv, out, tg, lse, dq, dk, dv)
        assert p.sync_status() == 0
        o_ref, lse_ref = oracle.forward(qr, kr, vr, H, scale, True, f64=True)
        assert np.abs(out.float().cpu().numpy() - o_ref).max() <= TOL_O_BF16
        assert np.abs(lse.cpu().numpy() - lse_ref).max() <= 2e-3
        for g, r in zip((dq, dk, dv), oracle.backward(qr, kr, vr, gr, H, scale, True, f64=True)):
            assert rel_err(g.float().cpu().numpy(), r) <= 2e-2
    finally:
        if created:
            dist.destroy_process_group()
