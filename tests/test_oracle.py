"""The oracle against the committed golden vectors and the reference's own known-answer tests.

CPU only. Tolerances: the reference's tests use 2e-4 absolute for the closed-form cases and
2e-3 for central finite differences (darkforest-cuda/src/lib.rs:2623, 2783, 2823).
"""
import math

import numpy as np
import pytest

from oracle import attn_oracle as ao


def _case(golden, name):
    idx = list(golden["cases"]).index(name)
    B, H, S, D, causal, seed = (int(x) for x in golden["case_params"][idx])
    return B, H, S, D, bool(causal), seed


def _inputs(oracle, B, H, S, D, seed):
    return tuple(oracle.fill_normal((B, S, H * D), seed, st) for st in range(4))


def test_reference_forward_known_answer(oracle, golden):
    q, k, v = golden["kat_fwd_q"], golden["kat_fwd_k"], golden["kat_fwd_v"]
    scale = 1.0 / math.sqrt(4.0)
    for f64 in (False, True):
        out, lse = oracle.forward(q, k, v, 1, scale, True, f64=f64)
        assert np.abs(out - golden["kat_fwd_out"]).max() <= 2e-4
        assert np.abs(lse - golden["kat_fwd_lse"]).max() <= 2e-4
    o_np, lse_np = ao.numpy_forward(q, k, v, 1, scale, True)
    assert np.abs(o_np - golden["kat_fwd_out"]).max() <= 1e-12
    assert np.abs(lse_np - golden["kat_fwd_lse"]).max() <= 1e-12


def test_reference_backward_known_answer_and_finite_difference(oracle, golden):
    q, k, v, go = (golden[f"kat_bwd_{n}"] for n in ("q", "k", "v", "do"))
    scale = 1.0 / math.sqrt(3.0)
    for f64 in (False, True):
        grads = oracle.backward(q, k, v, go, 1, scale, True, f64=f64)
        for g, n in zip(grads, ("dq", "dk", "dv")):
            assert np.abs(g - golden[f"kat_bwd_{n}"]).max() <= 2e-4, n
    # central differences of sum(O*dO), delta = 1e-3, tol 2e-3 (lib.rs:2785-2827)
    grads = oracle.backward(q, k, v, go, 1, scale, True)

    def objective(q_, k_, v_):
        out, _ = oracle.forward(q_, k_, v_, 1, scale, True)
        return float((out.astype(np.float64) * go).sum())

    delta = 1e-3
    for which, analytical in enumerate(grads):
        base = [q, k, v]
        flat = analytical.reshape(-1)
        for index in range(flat.size):
            plus = [a.copy() for a in base]
            minus = [a.copy() for a in base]
            plus[which].reshape(-1)[index] += delta
            minus[which].reshape(-1)[index] -= delta
            numerical = (objective(*plus) - objective(*minus)) / (2 * delta)
            assert abs(flat[index] - numerical) <= 2e-3


@pytest.mark.parametrize("name", ["mh_small", "mh_noncausal", "mh_d128", "mh_ragged", "mh_cfg1"])
def test_oracle_matches_golden_multihead(oracle, golden, name):
    B, H, S, D, causal, seed = _case(golden, name)
    q, k, v, go = _inputs(oracle, B, H, S, D, seed)
    rows = golden[f"{name}_rows"]
    scale = 1.0 / math.sqrt(D)
    for f64, tol in ((False, 2e-5), (True, 2e-6)):
        out, lse = oracle.forward(q, k, v, H, scale, causal, f64=f64)
        dq, dk, dv = oracle.backward(q, k, v, go, H, scale, causal, f64=f64)
        assert np.abs(out[:, rows] - golden[f"{name}_out"]).max() <= tol
        assert np.abs(lse[:, :, rows] - golden[f"{name}_lse"]).max() <= tol * 4
        for g, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            ref = golden[f"{name}_{n}"]
            assert np.abs(g[:, rows] - ref).max() <= tol * 10 * max(1.0, np.abs(ref).max()), n


def test_numpy_restatement_matches_c(oracle):
    B, H, S, D = 2, 3, 21, 12
    q, k, v, go = _inputs(oracle, B, H, S, D, 77)
    scale = 0.3
    for causal in (True, False):
        o_c, lse_c = oracle.forward(q, k, v, H, scale, causal, f64=True)
        o_n, lse_n = ao.numpy_forward(q, k, v, H, scale, causal)
        assert np.abs(o_c - o_n).max() < 1e-6 and np.abs(lse_c - lse_n).max() < 1e-6
        for a, b in zip(oracle.backward(q, k, v, go, H, scale, causal, f64=True),
                        ao.numpy_backward(q, k, v, go, H, scale, causal)):
            assert np.abs(a - b).max() < 2e-6


def test_seeded_generator_mirror_and_moments(oracle):
    a = oracle.fill_normal((4096,), 0xDF01, 2)
    b = ao.numpy_fill_normal(4096, 0xDF01, 2)
    assert np.abs(a - b).max() < 1e-6
    big = oracle.fill_normal((1 << 20,), 1, 0)
    assert abs(float(big.mean())) < 5e-3 and abs(float(big.std()) - 1.0) < 5e-3
    assert not np.array_equal(oracle.fill_normal((64,), 1, 0), oracle.fill_normal((64,), 1, 1))


def test_delta_and_merge(oracle):
    B, H, S, D = 1, 2, 37, 16
    q, k, v, go = _inputs(oracle, B, H, S, D, 5)
    scale = 0.25
    out, lse = oracle.forward(q, k, v, H, scale, True)
    d = oracle.delta(out, go, H)
    ref = (out.reshape(B, S, H, D).astype(np.float64) * go.reshape(B, S, H, D)).sum(-1).transpose(0, 2, 1)
    assert np.abs(d - ref).max() < 1e-5
    # split the keys in two halves (non-causal partials) and merge: equals attention over all keys
    half = S // 2
    qh = q
    s_all, lse_all = ao.numpy_forward(qh, k, v, H, scale, False)
    # partial over keys [0,half) and [half,S) computed with the numpy restatement on sliced K/V
    def part(ks, vs):
        B_, S_, dm = qh.shape
        qq = qh.reshape(B_, S_, H, D).transpose(0, 2, 1, 3).astype(np.float64)
        kk = ks.reshape(B_, -1, H, D).transpose(0, 2, 1, 3).astype(np.float64)
        vv = vs.reshape(B_, -1, H, D).transpose(0, 2, 1, 3).astype(np.float64)
        s = np.einsum("bhid,bhjd->bhij", qq, kk) * scale
        m = s.max(-1, keepdims=True)
        w = np.exp(s - m)
        l = w.sum(-1, keepdims=True)
        o = np.einsum("bhij,bhjd->bhid", w / l, vv).transpose(0, 2, 1, 3).reshape(B_, S_, H * D)
        return np.ascontiguousarray(o, np.float32), np.ascontiguousarray((m + np.log(l))[..., 0], np.float32)

    oa, la = part(k[:, :half], v[:, :half])
    ob, lb = part(k[:, half:], v[:, half:])
    om, lm = oracle.merge_partials(oa, la, ob, lb, H)
    assert np.abs(om - s_all).max() < 1e-5 and np.abs(lm - lse_all).max() < 1e-5
    # an empty partial (lse = -inf) leaves the other untouched
    empty_l = np.full_like(la, -np.inf)
    om2, lm2 = oracle.merge_partials(oa, la, np.zeros_like(oa), empty_l, H)
    assert np.array_equal(lm2, la) and np.abs(om2 - oa).max() < 1e-6


def test_edge_cases(oracle):
    # S = 1: the output is V, gradients of q and k vanish
    q, k, v, go = _inputs(oracle, 1, 2, 1, 8, 9)
    out, lse = oracle.forward(q, k, v, 2, 0.5, True)
    assert np.allclose(out, v)
    dq, dk, dv = oracle.backward(q, k, v, go, 2, 0.5, True)
    assert np.abs(dq).max() == 0 and np.abs(dk).max() == 0 and np.allclose(dv, go)
    # S = 0 is a no-op
    z = np.zeros((1, 0, 8), np.float32)
    out, lse = oracle.forward(z, z, z, 2, 0.5, True)
    assert out.size == 0


# ------------------------------------------------------------------ decode (one token over a KV cache)
def _decode_case(oracle, golden, name):
    idx = list(golden["dec_cases"]).index(name)
    H, D, T, T_max, seed = (int(x) for x in golden["dec_case_params"][idx])
    q = oracle.fill_normal((H * D,), seed, 0)
    k, v = (oracle.fill_normal((T_max, H * D), seed, st) for st in (1, 2))
    return H, D, T, T_max, q, k, v


@pytest.mark.parametrize("name", ["dec_small", "dec_d128", "dec_odd", "dec_cfg"])
def test_decode_oracle_matches_golden(oracle, golden, name):
    """C restatement of kernel_fused_mha_decode_kv (attention_fused.cu:551-615) and its paged form
    (:796-865) against torch float64 expectations."""
    from oracle.attn_oracle import numpy_decode
    H, D, T, T_max, q, k, v = _decode_case(oracle, golden, name)
    scale = 1.0 / np.sqrt(D)
    for f64, tol in ((False, 2e-5), (True, 2e-6)):
        out, lse = oracle.decode(q, k, v, H, T, scale, f64=f64)
        assert np.abs(out - golden[f"{name}_out"]).max() <= tol, (name, f64)
        assert np.abs(lse - golden[f"{name}_lse"]).max() <= tol * 4, (name, f64)
    o_np, lse_np = numpy_decode(q, k, v, H, T, scale)
    assert np.abs(o_np - golden[f"{name}_out"]).max() <= 1e-9
    # the same tokens scattered over a paged pool through a shuffled block table
    page = 16
    n_pages = T_max // page
    table = np.random.RandomState(7).permutation(n_pages).astype(np.int32)
    kp, vp = np.zeros_like(k), np.zeros_like(v)
    for lp in range(n_pages):
        kp[table[lp] * page:(table[lp] + 1) * page] = k[lp * page:(lp + 1) * page]
        vp[table[lp] * page:(table[lp] + 1) * page] = v[lp * page:(lp + 1) * page]
    out_p, _ = oracle.decode(q, kp, vp, H, T, scale, block_table=table, page_size=page)
    out_c, _ = oracle.decode(q, k, v, H, T, scale)
    assert np.array_equal(out_p, out_c)


def test_rope_and_position_interpolation_oracle_against_numpy(oracle):
    """The C restatements of kernel_apply_rope and kernel_pos_embed_interpolate
    (attention_fused.cu:1143-1166, 1098-1125) against float64 numpy formulas."""
    H, D, rows, pos0, base = 3, 10, 5, 17, 10000.0
    x = oracle.fill_normal((rows, H * D), 31, 0)
    got = oracle.apply_rope(x, pos0, H, D, base)
    xr = x.reshape(rows, H, D // 2, 2).astype(np.float64)
    i = np.arange(D // 2)
    ang = (pos0 + np.arange(rows))[:, None, None] * (base ** (-2.0 * i / D))[None, None, :]
    want = np.stack([xr[..., 0] * np.cos(ang) - xr[..., 1] * np.sin(ang), xr[..., 0] * np.sin(ang) + xr[..., 1] * np.cos(ang)], -1)
    assert np.abs(got.reshape(rows, H, D // 2, 2) - want).max() <= 2e-5
    # rotations preserve the norm of every pair, and position 0 is the identity
    assert np.allclose(np.linalg.norm(got.reshape(-1, 2), axis=1), np.linalg.norm(x.reshape(-1, 2), axis=1), rtol=1e-5)
    assert np.array_equal(oracle.apply_rope(x[:1], 0, H, D, base), x[:1])
    # single-precision pow (the reference's) stays within an ulp of the frequency: small positions agree
    assert np.abs(oracle.apply_rope(x, 3, H, D, base, single_pow=True) - oracle.apply_rope(x, 3, H, D, base)).max() <= 1e-5
    table = oracle.fill_normal((8, 6), 32, 0)
    assert np.array_equal(oracle.pos_embed_interpolate(table, 5, 8, 8), table[5])
    for pos, max_len in ((0, 20), (7, 20), (19, 20), (9, 8 + 3)):
        at = np.float32(pos) * (np.float32(7) / np.float32(max_len - 1))
        lo = int(at)
        hi = min(lo + 1, 7)
        w = np.float64(at) - lo
        want = (1 - w) * table[lo].astype(np.float64) + w * table[hi]
        assert np.abs(oracle.pos_embed_interpolate(table, pos, 8, max_len) - want).max() <= 1e-6, (pos, max_len)


def test_linear_restatement_matches_float64_goldens(oracle, golden):
    """cpu_linear (static_gpt2.rs:2717-2733) restated in C, against torch float64 expectations: the fp32 flavour
    within fp32 summation error of a 768-term dot product, the double-accumulating flavour to rounding."""
    for name, (rows, fin, fout, seed) in zip(golden["lin_cases"], golden["lin_case_params"]):
        x = oracle.fill_normal((int(rows), int(fin)), int(seed), 0)
        w = (oracle.fill_normal((int(fout), int(fin)), int(seed), 1) * 0.02).astype(np.float32)
        b = (oracle.fill_normal((int(fout),), int(seed), 2) * 0.02).astype(np.float32)
        r = oracle.fill_normal((int(rows), int(fout)), int(seed), 3)
        want, want_res = golden[f"{name}_out"], golden[f"{name}_out_res"]
        assert np.abs(oracle.linear(x, w, b) - want).max() <= 2e-5, name
        assert np.abs(oracle.linear(x, w, b, f64=True) - want).max() <= 2e-7, name
        assert np.abs(oracle.linear(x, w, b, residual=r, f64=True) - want_res).max() <= 5e-7, name
        assert np.abs(oracle.linear(x, w) - (want - b)).max() <= 2e-5, name


def test_chunked_cross_entropy_restatement_matches_float64_goldens(oracle, golden):
    """softmax.cu:325-394 / 415-462 restated in C, against torch float64 log-softmax expectations."""
    for name, (rows, cols, total_rows, seed) in zip(golden["ce_cases"], golden["ce_case_params"]):
        z = (oracle.fill_normal((int(rows), int(cols)), int(seed), 0) * 3.0).astype(np.float32)
        tg = golden[f"{name}_targets"]
        keep = golden[f"{name}_cols"]
        for f64, tol in ((False, 2e-6), (True, 2e-7)):
            probs, grad, loss = oracle.chunked_ce(z, tg, int(total_rows), train=True, f64=f64)
            assert abs(loss - float(golden[f"{name}_loss"])) <= 2e-5 * max(1.0, abs(float(golden[f"{name}_loss"]))), name
            want_p = golden[f"{name}_probs"]
            assert (np.abs(probs[:, keep] - want_p) <= tol * 0.05 + 1e-5 * np.abs(want_p)).all(), name
            assert np.abs(grad[:, keep] - golden[f"{name}_grad"]).max() <= 1e-5 / int(total_rows) + 1e-9, name
            _, _, loss_eval = oracle.chunked_ce(z, tg, int(total_rows), train=False, f64=f64)
            assert abs(loss_eval - loss) <= 2e-6 * max(1.0, abs(loss)), name
