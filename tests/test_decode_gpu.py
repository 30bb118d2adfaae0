"""One-token decode attention on the GPU through the C ABI against the CPU oracle, the golden
vectors and, when built, the reference's own decode kernels
(darkforest-cuda/kernels/attention_fused.cu:551-1090)."""
import os

import numpy as np
import pytest

from helpers import pkg, to_dev

pytestmark = pytest.mark.gpu

TOL = 2e-5  # fp32 arithmetic like the reference (exp2 with folded scale instead of __expf)


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch


def _paged(torch, k, v, page, seed):
    """Scatters the rows of a contiguous cache over a pool with a shuffled block table."""
    n_pages = k.shape[0] // page
    table = np.random.RandomState(seed).permutation(n_pages).astype(np.int32)
    kp, vp = np.zeros_like(k), np.zeros_like(v)
    for lp in range(n_pages):
        kp[table[lp] * page:(table[lp] + 1) * page] = k[lp * page:(lp + 1) * page]
        vp[table[lp] * page:(table[lp] + 1) * page] = v[lp * page:(lp + 1) * page]
    return kp, vp, table


@pytest.mark.parametrize("name", ["dec_small", "dec_d128", "dec_odd", "dec_cfg"])
def test_decode_matches_golden_in_every_form(torch_cuda, oracle, golden, name):
    torch = torch_cuda
    p = pkg()
    idx = list(golden["dec_cases"]).index(name)
    H, D, T, T_max, seed = (int(x) for x in golden["dec_case_params"][idx])
    q = oracle.fill_normal((H * D,), seed, 0)
    k, v = (oracle.fill_normal((T_max, H * D), seed, st) for st in (1, 2))
    scale = 1.0 / np.sqrt(D)
    tq, tk, tv = to_dev(q, k, v)
    want = golden[f"{name}_out"]
    # scratch-free form (cluster merge)
    out = p.decode(tq, tk, tv, H, T, scale)
    assert p.sync_status() == 0
    assert np.abs(out.cpu().numpy() - want).max() <= TOL, name
    # split form with caller scratch sized like the reference's chunk_size = 64
    chunks = (T + 63) // 64
    parts = (torch.empty(H * chunks, device="cuda"), torch.empty(H * chunks, device="cuda"),
             torch.empty(H * chunks * D, device="cuda"))
    out = p.decode(tq, tk, tv, H, T, scale, partials=parts, max_chunks=chunks)
    assert p.sync_status() == 0
    assert np.abs(out.cpu().numpy() - want).max() <= TOL, name
    # paged pool, both forms
    kp, vp, table = _paged(torch, k, v, 16, 11)
    tkp, tvp = to_dev(kp, vp)
    tt = torch.from_numpy(table).cuda()
    for kwargs in ({}, {"partials": parts, "max_chunks": chunks}):
        out = p.decode(tq, tkp, tvp, H, T, scale, block_table=tt, page_size=16, **kwargs)
        assert p.sync_status() == 0
        assert np.abs(out.cpu().numpy() - want).max() <= TOL, (name, bool(kwargs))
    # bf16 pool: compare with the oracle on the bf16-rounded cache
    kb, _ = oracle.round_bf16(kp)
    vb, _ = oracle.round_bf16(vp)
    ref, _ = oracle.decode(q, kb, vb, H, T, scale, block_table=table, page_size=16)
    out = p.decode(tq, tkp.to(torch.bfloat16), tvp.to(torch.bfloat16), H, T, scale, block_table=tt, page_size=16)
    assert p.sync_status() == 0
    assert np.abs(out.cpu().numpy() - ref).max() <= TOL, name


def test_decode_sweep_against_oracle(torch_cuda, oracle):
    """Sequence lengths around the chunking boundaries, head sizes on the vector and scalar paths,
    an unaligned cache slice, and every legacy symbol."""
    torch = torch_cuda
    p = pkg()
    L = p.lib()
    for H, D, T in [(1, 64, 1), (2, 64, 7), (12, 64, 129), (12, 64, 4097), (3, 128, 2050), (5, 20, 333), (2, 1, 17),
                    (16, 128, 20000), (12, 64, 40000), (5, 33, 60000)]:  # the last three are large enough for the split form
        T_max = ((T + 31) // 32) * 32
        q = oracle.fill_normal((H * D,), 4000 + T, 0)
        k, v = (oracle.fill_normal((T_max, H * D), 4000 + T, st) for st in (1, 2))
        scale = 1.0 / np.sqrt(D)
        ref, _ = oracle.decode(q, k, v, H, T, scale)
        tq, tk, tv = to_dev(q, k, v)
        out = torch.full((H * D,), 7.0, device="cuda")
        L.launch_fused_mha_decode_kv(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), H, T, D, scale)
        assert p.sync_status() == 0
        assert np.abs(out.cpu().numpy() - ref).max() <= TOL, (H, D, T)
        chunk = 256
        chunks = (T + chunk - 1) // chunk
        pm, pl = torch.empty(H * chunks, device="cuda"), torch.empty(H * chunks, device="cuda")
        po = torch.empty(H * chunks * D, device="cuda")
        out.fill_(7.0)
        L.launch_fused_mha_decode_kv_splitk(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), pm.data_ptr(), pl.data_ptr(),
                                            po.data_ptr(), out.data_ptr(), H, T, D, scale, chunk)
        assert p.sync_status() == 0
        assert np.abs(out.cpu().numpy() - ref).max() <= TOL, (H, D, T, "splitk")
        kp, vp, table = _paged(torch, k, v, 32, T)
        tkp, tvp = to_dev(kp, vp)
        tt = torch.from_numpy(table).cuda()
        out.fill_(7.0)
        L.launch_paged_mha_decode_kv(tq.data_ptr(), tkp.data_ptr(), tvp.data_ptr(), tt.data_ptr(), out.data_ptr(), H, T, D,
                                     scale, 32)
        assert np.abs(out.cpu().numpy() - ref).max() <= TOL, (H, D, T, "paged")
        out.fill_(7.0)
        L.launch_paged_mha_decode_kv_splitk(tq.data_ptr(), tkp.data_ptr(), tvp.data_ptr(), tt.data_ptr(), pm.data_ptr(),
                                            pl.data_ptr(), po.data_ptr(), out.data_ptr(), H, T, D, scale, 32, chunk)
        assert p.sync_status() == 0
        assert np.abs(out.cpu().numpy() - ref).max() <= TOL, (H, D, T, "paged splitk")
        kb, vb = oracle.round_bf16(kp)[0], oracle.round_bf16(vp)[0]
        ref16, _ = oracle.decode(q, kb, vb, H, T, scale, block_table=table, page_size=32)
        out.fill_(7.0)
        tkb, tvb = tkp.to(torch.bfloat16), tvp.to(torch.bfloat16)  # kept alive until the launch has been checked
        L.launch_paged_mha_decode_kv_bf16(tq.data_ptr(), tkb.data_ptr(), tvb.data_ptr(), tt.data_ptr(), out.data_ptr(), H, T, D,
                                          scale, 32)
        assert p.sync_status() == 0
        assert np.abs(out.cpu().numpy() - ref16).max() <= TOL, (H, D, T, "bf16")
    # cache slices that are only 4-byte aligned take the scalar loads
    H, D, T = 4, 64, 500
    q = oracle.fill_normal((H * D,), 77, 0)
    k, v = (oracle.fill_normal((512, H * D), 77, st) for st in (1, 2))
    ref, _ = oracle.decode(q, k, v, H, T, 0.125)
    big_k = torch.zeros(512 * H * D + 1, device="cuda")
    big_v = torch.zeros(512 * H * D + 1, device="cuda")
    big_k[1:] = torch.from_numpy(k).reshape(-1).cuda()
    big_v[1:] = torch.from_numpy(v).reshape(-1).cuda()
    out = p.decode(to_dev(q)[0], big_k[1:], big_v[1:], H, T, 0.125)
    assert p.sync_status() == 0
    assert np.abs(out.cpu().numpy() - ref).max() <= TOL
    # an empty cache leaves the output alone, like the reference kernels
    out = torch.full((H * D,), 7.0, device="cuda")
    L.launch_fused_mha_decode_kv(to_dev(q)[0].data_ptr(), big_k.data_ptr(), big_v.data_ptr(), out.data_ptr(), H, 0, D, 0.125)
    assert float(out.min()) == 7.0 and p.sync_status() == 0


def test_decode_matches_reference_cuda_kernels(torch_cuda, oracle):
    """The reference's own decode kernels, compiled unmodified for sm_100a, on the same inputs."""
    torch = torch_cuda
    from oracle.attn_oracle import ReferenceKernels, REFERENCE_SO
    if not os.path.exists(REFERENCE_SO):
        pytest.skip("oracle/_ref not built (reference tree absent when build() ran)")
    ref = ReferenceKernels()
    p = pkg()
    for H, D, T in [(12, 64, 1000), (4, 128, 3000), (3, 40, 257)]:
        q = oracle.fill_normal((H * D,), 5000 + T, 0)
        k, v = (oracle.fill_normal((T, H * D), 5000 + T, st) for st in (1, 2))
        scale = 1.0 / np.sqrt(D)
        tq, tk, tv = to_dev(q, k, v)
        want = ref.decode_kv(tq, tk, tv, H, T, scale).cpu().numpy()
        got = p.decode(tq, tk, tv, H, T, scale).cpu().numpy()
        cpu, _ = oracle.decode(q, k, v, H, T, scale)
        assert np.abs(got - want).max() <= TOL, (H, D, T)
        assert np.abs(cpu - want).max() <= TOL, (H, D, T)


# ------------------------------------------------------------------ per-token helpers of the same reference file
def test_rope_position_interpolation_and_paged_row_copies(torch_cuda, oracle):
    """launch_apply_rope, launch_pos_embed_interpolate, launch_paged_copy_row(_f32_to_bf16) and the batched
    rope against the oracle and, when built, against the reference's own kernels."""
    torch = torch_cuda
    p = pkg()
    L = p.lib()
    ref = None
    from oracle.attn_oracle import REFERENCE_SO
    if os.path.exists(REFERENCE_SO):
        import ctypes
        ref = ctypes.CDLL(REFERENCE_SO, mode=ctypes.RTLD_LOCAL)
    U, F, P = __import__("ctypes").c_uint32, __import__("ctypes").c_float, __import__("ctypes").c_void_p
    # rotary embedding: one row (legacy symbol), even and odd head sizes, and a block of rows
    for H, D, pos in [(12, 64, 0), (12, 64, 37), (4, 128, 1000), (3, 7, 5)]:
        x = oracle.fill_normal((H * D,), 600 + D, 0)
        t, = to_dev(x)
        L.launch_apply_rope(t.data_ptr(), pos, H, D, 10000.0)
        assert p.sync_status() == 0
        want = oracle.apply_rope(x.reshape(1, -1), pos, H, D, 10000.0).reshape(-1)
        assert np.abs(t.cpu().numpy() - want).max() <= 2e-5, (H, D, pos)
        if ref is not None:
            ref.launch_apply_rope.argtypes = [P, U, U, U, F]
            ref.launch_apply_rope.restype = None
            t2, = to_dev(x)
            ref.launch_apply_rope(t2.data_ptr(), pos, H, D, 10000.0)
            torch.cuda.synchronize()
            # the reference evaluates the frequency with powf: one ulp of it times the position
            assert np.abs(t.cpu().numpy() - t2.cpu().numpy()).max() <= 2e-5 + 4e-7 * pos * np.abs(x).max(), (H, D, pos)
    rows, H, D = 300, 12, 64
    x = oracle.fill_normal((rows, H * D), 77, 0)
    t, = to_dev(x)
    assert L.df_attn_apply_rope_rows(t.data_ptr(), 11, rows, H, D, 10000.0, None) == 0
    assert p.sync_status() == 0
    assert np.abs(t.cpu().numpy() - oracle.apply_rope(x, 11, H, D, 10000.0)).max() <= 2e-5
    # position-table interpolation: inside the trained range and stretched
    trained, dm = 64, 768
    table = oracle.fill_normal((trained, dm), 78, 0)
    tt, = to_dev(table)
    out = torch.empty(dm, device="cuda")
    for pos, max_len in [(5, 64), (63, 64), (0, 256), (100, 256), (255, 256), (64, 65)]:
        L.launch_pos_embed_interpolate(tt.data_ptr(), out.data_ptr(), pos, trained, max_len, dm)
        assert p.sync_status() == 0
        assert np.abs(out.cpu().numpy() - oracle.pos_embed_interpolate(table, pos, trained, max_len)).max() <= 1e-6, (pos, max_len)
        if ref is not None:
            ref.launch_pos_embed_interpolate.argtypes = [P, P, U, U, U, U]
            ref.launch_pos_embed_interpolate.restype = None
            out2 = torch.empty(dm, device="cuda")
            ref.launch_pos_embed_interpolate(tt.data_ptr(), out2.data_ptr(), pos, trained, max_len, dm)
            torch.cuda.synchronize()
            assert np.abs(out.cpu().numpy() - out2.cpu().numpy()).max() <= 1e-6, (pos, max_len)
    L.launch_pos_embed_interpolate(tt.data_ptr(), out.data_ptr(), 300, trained, 256, dm)  # beyond the stretched context
    assert L.df_attn_last_status() != 0
    p.sync_status()
    # row copies into a paged pool: bit-exact, bf16 rounded to nearest even, neighbours untouched
    page, n_pages = 16, 8
    row = oracle.fill_normal((dm,), 79, 0)
    tr, = to_dev(row)
    pool = torch.full((n_pages * page, dm), 7.0, device="cuda")
    L.launch_paged_copy_row(tr.data_ptr(), pool.data_ptr(), 5, 3, page, dm)
    assert p.sync_status() == 0
    got = pool.cpu().numpy()
    assert np.array_equal(got[5 * page + 3], row) and float(np.delete(got, 5 * page + 3, 0).min()) == 7.0
    pool16 = torch.zeros((n_pages * page, dm), device="cuda", dtype=torch.bfloat16)
    L.launch_paged_copy_row_f32_to_bf16(tr.data_ptr(), pool16.data_ptr(), 2, 15, page, dm)
    assert p.sync_status() == 0
    want16, _ = oracle.round_bf16(row)
    got16 = pool16.float().cpu().numpy()
    assert np.array_equal(got16[2 * page + 15], want16) and float(np.abs(np.delete(got16, 2 * page + 15, 0)).max()) == 0.0
    L.launch_paged_copy_row(tr.data_ptr(), pool.data_ptr(), 5, page, page, dm)  # offset outside the page
    assert L.df_attn_last_status() != 0
    p.sync_status()
