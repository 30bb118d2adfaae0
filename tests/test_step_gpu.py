"""GPU parity of the training step's LayerNorm, GELU and AdamW kernels, through the C ABI (df_* and the legacy launch_*
symbols), against the CPU oracle, the float64 golden vectors and the reference's own kernels compiled unmodified.
fp32 arithmetic like the reference; tolerances: LayerNorm output and grad_x 2e-5 of the tensor's scale (sums run in a
different order), grad_gamma / grad_beta 2e-5 of their scale times sqrt(rows); GELU 2e-6 absolute per unit of |x|
(one exponential instead of tanhf); AdamW 1e-6 absolute on parameters of order 1 (the reference's own bar) and
equal to the reference kernel to 2 ulp."""
import os

import numpy as np
import pytest

from helpers import ROOT, pkg, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "these tests need a GPU"
    torch.cuda.set_device(0)
    p = pkg()
    p.lib()
    yield torch
    assert p.sync_status() == 0


@pytest.fixture(scope="module")
def step_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "step_golden.npz"))


def _ln_inputs(oracle, rows, cols, seed):
    x = (oracle.fill_normal((rows, cols), seed, 0) * 1.7 + 0.3).astype(np.float32)
    gamma = (1.0 + 0.2 * oracle.fill_normal((cols,), seed, 1)).astype(np.float32)
    beta = (0.1 * oracle.fill_normal((cols,), seed, 2)).astype(np.float32)
    go = oracle.fill_normal((rows, cols), seed, 3).astype(np.float32)
    return x, gamma, beta, go


# widths: below one vector, ragged (scalar kernels), the model width 768 (six float4 per lane), 1024 (eight), wider than a
# warp's registers forward (1600, 4096) and beyond that (5000); rows: one, fewer than a block's warps, more than the grid
@pytest.mark.parametrize("rows,cols", [(1, 1), (1, 3), (3, 50), (5, 12), (9, 768), (300, 768), (4096, 768), (33, 1024), (7, 1600),
                                       (2, 4096), (3, 5000), (40000, 64)])
def test_layernorm_forward_backward_match_oracle(torch_cuda, oracle, rows, cols):
    torch = torch_cuda
    p = pkg()
    x, gamma, beta, go = _ln_inputs(oracle, rows, cols, 7000 + rows + cols)
    tx, tg, tb, tgo = to_dev(x, gamma, beta, go)
    out, means, rstds = p.layernorm(tx, tg, tb)
    o_ref, m_ref, r_ref = oracle.layernorm(x, gamma, beta, f64=True)
    scale = max(1.0, np.abs(o_ref).max())
    assert np.abs(out.cpu().numpy() - o_ref).max() <= 2e-5 * scale
    assert np.abs(means.cpu().numpy() - m_ref).max() <= 2e-6 * max(1.0, np.abs(m_ref).max())
    assert np.abs(rstds.cpu().numpy() / r_ref - 1).max() <= 2e-5
    # backward from the kernel's own statistics; the column sums are added to what the buffers hold
    gg = torch.full((cols,), 0.5, device="cuda")
    gb = torch.full((cols,), -0.25, device="cuda")
    gx = p.layernorm_backward(tgo, tx, tg, means, rstds, grad_gamma=gg, grad_beta=gb)
    assert p.sync_status() == 0
    gx_ref, gg_ref, gb_ref = oracle.layernorm_backward(go, x, gamma, m_ref, r_ref, f64=True)
    assert np.abs(gx.cpu().numpy() - gx_ref).max() <= 2e-5 * max(1.0, np.abs(gx_ref).max())
    col_tol = 2e-5 * np.sqrt(rows)
    assert np.abs(gg.cpu().numpy() - 0.5 - gg_ref).max() <= col_tol * max(1.0, np.abs(gg_ref).max())
    assert np.abs(gb.cpu().numpy() + 0.25 - gb_ref).max() <= col_tol * max(1.0, np.abs(gb_ref).max())


@pytest.mark.parametrize("rows,cols", [(4096, 768), (2400, 1024), (40000, 64), (2368, 4), (5000, 1000)])
def test_layernorm_backward_staged_and_register_forms(torch_cuda, oracle, rows, cols):
    """With enough rows to fill the machine the backward stages its rows in shared memory with bulk copies (option
    OPT_LN_STAGED, default on); the same shapes through the register form and through the staged form, both against
    the oracle: 16 and 8 warps per block, 2 to 4 rows in flight per warp, rows far shorter than a warp."""
    torch = torch_cuda
    p = pkg()
    x, gamma, beta, go = _ln_inputs(oracle, rows, cols, 7600 + cols)
    tx, tg, tgo = to_dev(x, gamma, go)
    _, m_ref, r_ref = oracle.layernorm(x, gamma, beta, f64=True)
    tm, tr = to_dev(m_ref, r_ref)
    gx_ref, gg_ref, gb_ref = oracle.layernorm_backward(go, x, gamma, m_ref, r_ref, f64=True)
    for staged in (1, 0):
        prev = p.set_option(p.OPT_LN_STAGED, staged)
        try:
            gg, gb = torch.zeros(cols, device="cuda"), torch.zeros(cols, device="cuda")
            gx = p.layernorm_backward(tgo, tx, tg, tm, tr, grad_gamma=gg, grad_beta=gb)
            assert p.sync_status() == 0
        finally:
            p.set_option(p.OPT_LN_STAGED, prev)
        assert np.abs(gx.cpu().numpy() - gx_ref).max() <= 2e-5 * max(1.0, np.abs(gx_ref).max()), staged
        col_tol = 2e-5 * np.sqrt(rows)
        assert np.abs(gg.cpu().numpy() - gg_ref).max() <= col_tol * max(1.0, np.abs(gg_ref).max()), staged
        assert np.abs(gb.cpu().numpy() - gb_ref).max() <= col_tol * max(1.0, np.abs(gb_ref).max()), staged


def test_layernorm_optional_arguments_and_misaligned_rows(torch_cuda, oracle):
    """gamma / beta / means / rstds / grad_gamma / grad_beta absent; a matrix that starts 4 bytes off a 16-byte boundary
    takes the scalar kernels and gives the same result."""
    torch = torch_cuda
    p = pkg()
    rows, cols = 37, 768
    x, gamma, beta, go = _ln_inputs(oracle, rows, cols, 7100)
    tx, tgo = to_dev(x, go)
    out = torch.empty_like(tx)
    assert p.lib().df_layernorm_forward(tx.data_ptr(), None, None, out.data_ptr(), None, None, rows, cols, None) == 0
    o_ref, m_ref, r_ref = oracle.layernorm(x, f64=True)
    assert np.abs(out.cpu().numpy() - o_ref).max() <= 2e-5 * max(1.0, np.abs(o_ref).max())
    tm, tr = to_dev(m_ref, r_ref)
    gx = p.layernorm_backward(tgo, tx, None, tm, tr)
    gx_ref, _, _ = oracle.layernorm_backward(go, x, None, m_ref, r_ref, f64=True)
    assert np.abs(gx.cpu().numpy() - gx_ref).max() <= 2e-5 * max(1.0, np.abs(gx_ref).max())
    # misaligned: views one float into larger buffers
    bx, bo, bg = (torch.empty(rows * cols + 1, device="cuda") for _ in range(3))
    vx, vo, vg = bx[1:].view(rows, cols), bo[1:].view(rows, cols), bg[1:].view(rows, cols)
    vx.copy_(tx)
    vg.copy_(tgo)
    L = p.lib()
    assert L.df_layernorm_forward(vx.data_ptr(), None, None, vo.data_ptr(), tm.data_ptr(), tr.data_ptr(), rows, cols, None) == 0
    assert np.abs(vo.cpu().numpy() - o_ref).max() <= 2e-5 * max(1.0, np.abs(o_ref).max())
    assert L.df_layernorm_backward(vg.data_ptr(), vx.data_ptr(), None, tm.data_ptr(), tr.data_ptr(), vo.data_ptr(), None, None,
                                   rows, cols, None) == 0
    assert np.abs(vo.cpu().numpy() - gx_ref).max() <= 2e-5 * max(1.0, np.abs(gx_ref).max())
    # empty inputs are no-ops, missing required pointers are refused on the host
    assert L.df_layernorm_forward(None, None, None, None, None, None, 0, 768, None) == 0
    assert L.df_layernorm_forward(None, None, None, out.data_ptr(), None, None, 4, 768, None) == p.DF_ERR_INVALID_ARG
    assert L.df_gelu_forward(None, None, 0, None) == 0
    assert L.df_adamw_update(tx.data_ptr(), tx.data_ptr(), tx.data_ptr(), tx.data_ptr(), 8, 1e-3, 0.9, 0.999, 1e-8, 0.0, 0.0, 1.0,
                             None) == p.DF_ERR_INVALID_ARG   # a zero bias correction would divide by zero
    p.lib().df_attn_last_status()


def test_layernorm_golden_and_legacy_symbols(torch_cuda, oracle, step_golden):
    torch = torch_cuda
    p = pkg()
    L = p.lib()
    g = step_golden
    for name, (rows, cols, seed) in zip(g["ln_cases"], g["ln_case_params"]):
        rows, cols = int(rows), int(cols)
        x, gamma, beta, go = _ln_inputs(oracle, rows, cols, int(seed))
        tx, tg, tb, tgo = to_dev(x, gamma, beta, go)
        out, gx = torch.empty_like(tx), torch.empty_like(tx)
        means, rstds = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
        gg, gb = torch.zeros(cols, device="cuda"), torch.zeros(cols, device="cuda")
        L.launch_layernorm(tx.data_ptr(), tg.data_ptr(), tb.data_ptr(), out.data_ptr(), means.data_ptr(), rstds.data_ptr(), rows, cols)
        L.launch_layernorm_backward(tgo.data_ptr(), tx.data_ptr(), tg.data_ptr(), means.data_ptr(), rstds.data_ptr(), gx.data_ptr(),
                                    gg.data_ptr(), gb.data_ptr(), rows, cols)
        L.darkforest_sync()
        assert np.abs(out.cpu().numpy() - g[f"{name}_out"]).max() <= 2e-5 * max(1.0, np.abs(g[f"{name}_out"]).max()), name
        assert np.abs(gx.cpu().numpy() - g[f"{name}_gx"]).max() <= 2e-5 * max(1.0, np.abs(g[f"{name}_gx"]).max()), name
        assert np.abs(gg.cpu().numpy() - g[f"{name}_ggamma"]).max() <= 4e-5 * max(1.0, np.abs(g[f"{name}_ggamma"]).max()), name
        assert np.abs(gb.cpu().numpy() - g[f"{name}_gbeta"]).max() <= 4e-5 * max(1.0, np.abs(g[f"{name}_gbeta"]).max()), name


@pytest.mark.parametrize("n", [1, 3, 4, 5, 1023, 4099, 1 << 20, (1 << 22) + 3])
def test_gelu_matches_oracle(torch_cuda, oracle, n):
    torch = torch_cuda
    p = pkg()
    x = (oracle.fill_normal((n,), 7200 + n % 97, 0) * 3.0).astype(np.float32)
    x[: min(n, 6)] = np.array([-30.0, 30.0, 0.0, -8.0, 8.0, 1e-20], np.float32)[: min(n, 6)]   # saturated tails, zero
    go = oracle.fill_normal((n,), 7200 + n % 97, 1).astype(np.float32)
    tx, tgo = to_dev(x, go)
    y = p.gelu(tx)
    gx = p.gelu_backward(tgo, tx)
    assert p.sync_status() == 0
    y_ref, gx_ref = oracle.gelu(x, f64=True), oracle.gelu_backward(go, x, f64=True)
    assert np.isfinite(y.cpu().numpy()).all() and np.isfinite(gx.cpu().numpy()).all()
    assert (np.abs(y.cpu().numpy() - y_ref) <= 2e-6 * np.maximum(1.0, np.abs(x))).all()
    assert (np.abs(gx.cpu().numpy() - gx_ref) <= 4e-6 * np.maximum(1.0, np.abs(x)) * np.maximum(1.0, np.abs(go))).all()
    # a misaligned view takes the scalar kernel
    if n > 8:
        y2 = torch.empty(n, device="cuda")
        assert p.lib().df_gelu_forward(tx[1:].data_ptr(), y2.data_ptr(), n - 1, None) == 0
        assert torch.equal(y2[: n - 1], y[1:])


def test_gelu_golden_and_legacy_symbols(torch_cuda, oracle, step_golden):
    torch = torch_cuda
    p = pkg()
    L = p.lib()
    g = step_golden
    n, seed = (int(a) for a in g["gelu_params"])
    x = (oracle.fill_normal((n,), seed, 0) * 2.5).astype(np.float32)
    x[:5] = [-2.0, -1.0, 0.0, 1.0, 2.0]
    go = oracle.fill_normal((n,), seed, 1).astype(np.float32)
    tx, tgo = to_dev(x, go)
    y, gx = torch.empty_like(tx), torch.empty_like(tx)
    L.launch_gelu(tx.data_ptr(), y.data_ptr(), n)
    L.launch_gelu_backward(tgo.data_ptr(), tx.data_ptr(), gx.data_ptr(), n)
    L.darkforest_sync()
    assert np.abs(y.cpu().numpy() - g["gelu_out"]).max() <= 1e-5     # the reference's own bar, lib.rs:2832-2848
    assert np.abs(gx.cpu().numpy() - g["gelu_gx"]).max() <= 2e-5


def _adam_case(oracle, n, seed):
    return (oracle.fill_normal((n,), seed, 0), (0.1 * oracle.fill_normal((n,), seed, 1)).astype(np.float32),
            (0.01 * oracle.fill_normal((n,), seed, 2) ** 2).astype(np.float32), oracle.fill_normal((n,), seed, 3))


@pytest.mark.parametrize("n", [1, 3, 4, 7, 2048, 2049, 100003, 3 * 768 * 768])
def test_adamw_matches_oracle(torch_cuda, oracle, n):
    torch = torch_cuda
    p = pkg()
    hyper = (3e-4, 0.9, 0.999, 1e-8, 0.1, 1 - 0.9 ** 3, 1 - 0.999 ** 3)
    pp, mm, vv, gg = _adam_case(oracle, n, 7300 + n % 89)
    tp, tm, tv, tg = to_dev(pp, mm, vv, gg)
    p.adamw_update(tp, tm, tv, tg, *hyper)
    assert p.sync_status() == 0
    p_ref, m_ref, v_ref = oracle.adamw(pp, mm, vv, gg, *hyper)
    assert np.abs(tp.cpu().numpy() - p_ref).max() <= 1e-6
    assert np.abs(tm.cpu().numpy() - m_ref).max() <= 1e-7
    assert np.abs(tv.cpu().numpy() - v_ref).max() <= 1e-7
    assert torch.equal(tg, to_dev(gg)[0])


def test_adamw_golden_two_steps_and_legacy_symbol(torch_cuda, oracle, step_golden):
    torch = torch_cuda
    p = pkg()
    L = p.lib()
    g = step_golden
    n, seed = (int(a) for a in g["adamw_params"])
    lr, b1, b2, eps, wd = (float(a) for a in g["adamw_hyper"])
    tp = to_dev(oracle.fill_normal((n,), seed, 0))[0]
    tm, tv = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for t in (1, 2):
        tg = to_dev(oracle.fill_normal((n,), seed, t))[0]
        L.launch_adamw_update(tp.data_ptr(), tm.data_ptr(), tv.data_ptr(), tg.data_ptr(), n, lr, b1, b2, eps, wd, 1 - b1 ** t, 1 - b2 ** t)
        L.darkforest_sync()
        assert np.abs(tp.cpu().numpy() - g[f"adamw_p{t}"]).max() <= 1e-6   # the reference's own bar, lib.rs:2679-2751
        assert np.abs(tm.cpu().numpy() - g[f"adamw_m{t}"]).max() <= 5e-7


def test_adamw_multi_tensor_equals_per_tensor(torch_cuda, oracle):
    """One launch over a table of tensors (sizes around the 2048-element work unit, odd sizes, one tensor that starts
    4 bytes off a 16-byte boundary) gives bit-identical results to one df_adamw_update per tensor."""
    torch = torch_cuda
    p = pkg()
    hyper = (1e-3, 0.9, 0.95, 1e-8, 0.01, 1 - 0.9 ** 5, 1 - 0.95 ** 5)
    sizes = [1, 5, 2047, 2048, 2049, 768, 768 * 768, 50257 * 3 + 1, 4096, 3]
    single, multi = [], []
    for i, n in enumerate(sizes):
        arrs = _adam_case(oracle, n, 7400 + i)
        single.append(list(to_dev(*arrs)))
        if i == 4:   # misaligned copies: views one float into larger buffers
            bufs = [torch.empty(n + 1, device="cuda") for _ in range(4)]
            views = [b[1:] for b in bufs]
            for v, a in zip(views, to_dev(*arrs)):
                v.copy_(a)
            multi.append(views)
        else:
            multi.append(list(to_dev(*arrs)))
    for t in single:
        p.adamw_update(*t, *hyper)
    plan = p.AdamwPlan(multi)
    assert plan.total_chunks == sum((n + 2047) // 2048 for n in sizes)
    before = p.launch_count()
    plan.step(*hyper)
    assert p.launch_count() - before == 1
    assert p.sync_status() == 0
    for a, b in zip(single, multi):
        for x, y in zip(a[:3], b[:3]):
            assert torch.equal(x, y)
        assert torch.equal(a[3], b[3])


def test_step_kernels_match_reference_cuda_kernels(torch_cuda, oracle):
    """The reference's own kernels (layernorm.cu, elementwise.cu, matmul.cu compiled unmodified for sm_100a) on the same
    inputs: LayerNorm and GELU within the tolerances above, AdamW to 2 ulp."""
    torch = torch_cuda
    from oracle.attn_oracle import REFERENCE_SO, ReferenceKernels
    if not os.path.exists(REFERENCE_SO):
        pytest.skip("reference kernels not built")
    ref = ReferenceKernels()
    if not ref.has_step:
        pytest.skip("reference build without the step kernels")
    p = pkg()
    R = ref.lib
    rows, cols = 515, 768
    x, gamma, beta, go = _ln_inputs(oracle, rows, cols, 7500)
    tx, tg, tb, tgo = to_dev(x, gamma, beta, go)
    out, means, rstds = p.layernorm(tx, tg, tb)
    gg, gb = torch.zeros(cols, device="cuda"), torch.zeros(cols, device="cuda")
    gx = p.layernorm_backward(tgo, tx, tg, means, rstds, grad_gamma=gg, grad_beta=gb)
    r_out, r_gx = torch.empty_like(tx), torch.empty_like(tx)
    r_m, r_r = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    r_gg, r_gb = torch.zeros(cols, device="cuda"), torch.zeros(cols, device="cuda")
    torch.cuda.synchronize()
    R.launch_layernorm(tx.data_ptr(), tg.data_ptr(), tb.data_ptr(), r_out.data_ptr(), r_m.data_ptr(), r_r.data_ptr(), rows, cols)
    R.launch_layernorm_backward(tgo.data_ptr(), tx.data_ptr(), tg.data_ptr(), r_m.data_ptr(), r_r.data_ptr(), r_gx.data_ptr(),
                                r_gg.data_ptr(), r_gb.data_ptr(), rows, cols)
    torch.cuda.synchronize()
    assert float((out - r_out).abs().max()) <= 2e-5 * max(1.0, float(r_out.abs().max()))
    assert float((gx - r_gx).abs().max()) <= 2e-5 * max(1.0, float(r_gx.abs().max()))
    assert float((gg - r_gg).abs().max()) <= 2e-5 * np.sqrt(rows) * max(1.0, float(r_gg.abs().max()))
    assert float((gb - r_gb).abs().max()) <= 2e-5 * np.sqrt(rows) * max(1.0, float(r_gb.abs().max()))
    n = 100003
    xv = to_dev((oracle.fill_normal((n,), 7501, 0) * 3.0).astype(np.float32))[0]
    gv = to_dev(oracle.fill_normal((n,), 7501, 1))[0]
    y, dy = p.gelu(xv), p.gelu_backward(gv, xv)
    r_y, r_dy = torch.empty_like(xv), torch.empty_like(xv)
    torch.cuda.synchronize()
    R.launch_gelu(xv.data_ptr(), r_y.data_ptr(), n)
    R.launch_gelu_backward(gv.data_ptr(), xv.data_ptr(), r_dy.data_ptr(), n)
    torch.cuda.synchronize()
    assert bool(((y - r_y).abs() <= 2e-6 * xv.abs().clamp(min=1.0)).all())
    assert bool(((dy - r_dy).abs() <= 4e-6 * xv.abs().clamp(min=1.0) * gv.abs().clamp(min=1.0)).all())
    hyper = (3e-4, 0.9, 0.999, 1e-8, 0.1, 1 - 0.9 ** 2, 1 - 0.999 ** 2)
    arrs = _adam_case(oracle, n, 7502)
    mine, theirs = list(to_dev(*arrs)), list(to_dev(*arrs))
    p.adamw_update(*mine, *hyper)
    torch.cuda.synchronize()
    R.launch_adamw_update(*(t.data_ptr() for t in theirs), n, *hyper)
    torch.cuda.synchronize()
    for a, b in zip(mine[:3], theirs[:3]):
        ulp = torch.abs(a.view(torch.int32) - b.view(torch.int32)).max()
        assert int(ulp) <= 2
