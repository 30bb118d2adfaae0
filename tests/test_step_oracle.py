"""Pins the oracle's LayerNorm, GELU and AdamW restatements (CPU only): against the reference's own known-answer tests
(darkforest-cuda/src/lib.rs:2679-2751 AdamW one and two steps, tolerance 1e-6; :2832-2848 GELU at five points, 1e-5) and
against float64 vectors computed by torch (tests/golden/step_golden.npz, written by tests/golden/make_golden.py)."""
import math
import os

import numpy as np
import pytest

from helpers import ROOT


@pytest.fixture(scope="module")
def step_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "step_golden.npz"))


def _ln_inputs(oracle, rows, cols, seed):
    x = (oracle.fill_normal((rows, cols), seed, 0) * 1.7 + 0.3).astype(np.float32)
    gamma = (1.0 + 0.2 * oracle.fill_normal((cols,), seed, 1)).astype(np.float32)
    beta = (0.1 * oracle.fill_normal((cols,), seed, 2)).astype(np.float32)
    go = oracle.fill_normal((rows, cols), seed, 3).astype(np.float32)
    return x, gamma, beta, go


def test_gelu_known_answers_of_the_reference(oracle):
    x = np.array([-2.0, -1.0, 0.0, 1.0, 2.0], np.float32)
    c = math.sqrt(2.0 / math.pi)
    expected = np.array([0.5 * v * (1.0 + math.tanh(c * (v + 0.044715 * v ** 3))) for v in x])
    for f64 in (False, True):
        assert np.abs(oracle.gelu(x, f64=f64) - expected).max() <= 1e-5


def test_adamw_known_answers_of_the_reference(oracle):
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    grads = [np.array([0.2, -0.4, 0.8]), np.array([-0.1, 0.3, 0.2])]
    exp_p, exp_m, exp_v = np.array([1.0, -2.0, 0.5]), np.zeros(3), np.zeros(3)
    p, m, v = exp_p.astype(np.float32), np.zeros(3, np.float32), np.zeros(3, np.float32)
    for t, g in enumerate(grads, 1):
        exp_m = b1 * exp_m + (1 - b1) * g
        exp_v = b2 * exp_v + (1 - b2) * g * g
        exp_p = exp_p * (1 - lr * wd) - lr * (exp_m / (1 - b1 ** t)) / (np.sqrt(exp_v / (1 - b2 ** t)) + eps)
        p, m, v = oracle.adamw(p, m, v, g, lr, b1, b2, eps, wd, 1 - b1 ** t, 1 - b2 ** t)
        assert np.abs(p - exp_p).max() <= 1e-6, t
    # first step in closed form, as the reference writes it: m_hat = g, v_hat = g^2
    g = grads[0]
    first = np.array([1.0, -2.0, 0.5]) * (1 - lr * wd) - lr * g / (np.abs(g) + eps)
    p1, _, _ = oracle.adamw([1.0, -2.0, 0.5], np.zeros(3), np.zeros(3), g, lr, b1, b2, eps, wd, 1 - b1, 1 - b2)
    assert np.abs(p1 - first).max() <= 1e-6


def test_layernorm_against_float64(oracle, step_golden):
    g = step_golden
    for name, (rows, cols, seed) in zip(g["ln_cases"], g["ln_case_params"]):
        x, gamma, beta, go = _ln_inputs(oracle, int(rows), int(cols), int(seed))
        for f64, tol in ((True, 2e-6), (False, 2e-5)):
            out, means, rstds = oracle.layernorm(x, gamma, beta, f64=f64)
            assert np.abs(out - g[f"{name}_out"]).max() <= tol * 4, (name, f64)
            assert np.abs(means - g[f"{name}_mean"]).max() <= tol
            assert np.abs(rstds / g[f"{name}_rstd"] - 1).max() <= tol
            gx, gg, gb = oracle.layernorm_backward(go, x, gamma, means, rstds, f64=f64)
            assert np.abs(gx - g[f"{name}_gx"]).max() <= tol * 4 * max(1.0, np.abs(g[f"{name}_gx"]).max()), (name, f64)
            assert np.abs(gg - g[f"{name}_ggamma"]).max() <= tol * 4 * max(1.0, np.abs(g[f"{name}_ggamma"]).max())
            assert np.abs(gb - g[f"{name}_gbeta"]).max() <= tol * 4 * max(1.0, np.abs(g[f"{name}_gbeta"]).max())
    # no gamma / beta: plain normalisation; the column sums add to what the buffers hold
    x, gamma, beta, go = _ln_inputs(oracle, 4, 20, 99)
    out, means, rstds = oracle.layernorm(x)
    assert np.abs(out.mean(1)).max() <= 1e-6 and np.abs(out.var(1) - 1).max() <= 1e-3
    _, gg0, gb0 = oracle.layernorm_backward(go, x, gamma, means, rstds)
    _, gg1, gb1 = oracle.layernorm_backward(go, x, gamma, means, rstds, grad_gamma0=np.full(20, 2.0), grad_beta0=np.full(20, -1.0))
    assert np.allclose(gg1, gg0 + 2.0, atol=1e-6) and np.allclose(gb1, gb0 - 1.0, atol=1e-6)


def test_gelu_and_adamw_against_float64(oracle, step_golden):
    g = step_golden
    n, seed = (int(a) for a in g["gelu_params"])
    x = (oracle.fill_normal((n,), seed, 0) * 2.5).astype(np.float32)
    x[:5] = [-2.0, -1.0, 0.0, 1.0, 2.0]
    go = oracle.fill_normal((n,), seed, 1).astype(np.float32)
    for f64, tol in ((True, 5e-7), (False, 2e-6)):
        assert np.abs(oracle.gelu(x, f64=f64) - g["gelu_out"]).max() <= tol * 8
        assert np.abs(oracle.gelu_backward(go, x, f64=f64) - g["gelu_gx"]).max() <= tol * 8
    n, seed = (int(a) for a in g["adamw_params"])
    lr, b1, b2, eps, wd = (float(a) for a in g["adamw_hyper"])
    p = oracle.fill_normal((n,), seed, 0)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    for t in (1, 2):
        grad = oracle.fill_normal((n,), seed, t)
        p, m, v = oracle.adamw(p, m, v, grad, lr, b1, b2, eps, wd, 1 - b1 ** t, 1 - b2 ** t)
        assert np.abs(p - g[f"adamw_p{t}"]).max() <= 1e-6
        assert np.abs(m - g[f"adamw_m{t}"]).max() <= 5e-7   # 1 - 0.9f carries 2.4e-7 relative
        # 1 - 0.999f is 0.00100004673 in fp32: the second moment carries that 4.7e-5 relative offset by definition
        assert (np.abs(v - g[f"adamw_v{t}"]) <= 1e-4 * np.abs(g[f"adamw_v{t}"]) + 1e-9).all()


def test_adamw_plan_is_host_only_and_counts_work_units():
    """df_adamw_plan runs on the host (no GPU call): it numbers the 2048-element work units of a tensor table."""
    import ctypes
    from helpers import pkg
    p = pkg()
    sizes = [1, 2047, 2048, 2049, 0, 768 * 768, 5]
    table = (p.AdamwTensor * len(sizes))()
    for e, n in zip(table, sizes):
        e.n = n
    total = int(p.lib().df_adamw_plan(ctypes.cast(table, ctypes.c_void_p), len(sizes)))
    chunks = [(n + 2047) // 2048 for n in sizes]
    assert total == sum(chunks)
    assert [int(e.first_chunk) for e in table] == [sum(chunks[:i]) for i in range(len(sizes))]
    assert int(p.lib().df_adamw_plan(None, 3)) == 0
