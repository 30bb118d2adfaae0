"""The checked build of the library (make EXTRA=-DDF_BOUNDS_CHECK): the SIMT kernels range-check every global index.

The test builds that variant into a scratch directory (nvcc, about a minute), runs ragged shapes through the SIMT
path in a child process and expects (a) the same results as the oracle, (b) a clean device status word, and (c) that
the checker's own self-test - one thread asking for element 5 of a 4-element tensor - is reported as
DF_ERR_DEVICE_BOUNDS exactly once while the context stays usable. No out-of-range access is made anywhere."""
import json
import os
import shutil
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import json, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    import torch
    from __graft_entry__ import load_package
    from oracle.attn_oracle import Oracle, build
    pkg = load_package()
    pkg.LIB_PATH = {lib!r}
    build()
    orc = Oracle()
    res = {{"normal_build_refuses": None, "cases": []}}
    L = pkg.lib()
    prev = pkg.set_variant(pkg.VARIANT_SIMT)
    rng = np.random.default_rng(11)
    for (B, H, S, D, causal) in ((1, 1, 5, 4, True), (2, 3, 33, 3, True), (1, 2, 129, 64, True), (1, 2, 77, 128, False), (1, 12, 257, 32, True)):
        q, k, v, go = (rng.standard_normal((B, S, H * D), dtype=np.float32) for _ in range(4))
        tq, tk, tv, tg = (torch.from_numpy(x).cuda() for x in (q, k, v, go))
        scale = 1.0 / np.sqrt(D)
        out, lse = pkg.forward(tq, tk, tv, H, scale, causal)
        dq, dk, dv = pkg.backward(tq, tk, tv, out, tg, lse, H, scale, causal)
        st = pkg.sync_status()
        o_ref, lse_ref = orc.forward(q, k, v, H, scale, causal)
        dq_ref, dk_ref, dv_ref = orc.backward(q, k, v, go, H, scale, causal)
        res["cases"].append({{"shape": [B, H, S, D], "status": st,
                             "err_o": float(np.abs(out.cpu().numpy() - o_ref).max()),
                             "err_dq": float(np.abs(dq.cpu().numpy() - dq_ref).max()),
                             "err_dk": float(np.abs(dk.cpu().numpy() - dk_ref).max()),
                             "err_dv": float(np.abs(dv.cpu().numpy() - dv_ref).max())}})
    pkg.set_variant(prev)
    res["selftest_launch"] = L.df_attn_selftest_bounds_check(None)
    res["status_after_selftest"] = pkg.sync_status()
    res["status_again"] = pkg.sync_status()
    # the context is still usable
    q = torch.randn((1, 64, 2 * 64), device="cuda")
    out, _ = pkg.forward(q, q, q, 2, 0.125, True)
    res["status_after_forward"] = pkg.sync_status()
    res["finite"] = bool(torch.isfinite(out).all().item())
    print("RESULT " + json.dumps(res))
""")


@pytest.mark.gpu
def test_checked_build_runs_clean_and_reports_a_bad_index(tmp_path):
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("nvcc is not available: the checked variant cannot be built here")
    out_dir = str(tmp_path / "lib_checked")
    lib = os.path.join(out_dir, "libdarkforest_kernels.so")
    r = subprocess.run(["make", "-C", os.path.join(ROOT, "dark-forest_b200"), "-j8", f"OUT={out_dir}", "EXTRA=-DDF_BOUNDS_CHECK", lib],
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    child = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT, lib=lib)], capture_output=True, text=True, timeout=600)
    assert child.returncode == 0, child.stdout[-3000:] + child.stderr[-3000:]
    line = [l for l in child.stdout.splitlines() if l.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    for c in res["cases"]:
        assert c["status"] == 0, c
        assert max(c["err_o"], c["err_dq"], c["err_dk"], c["err_dv"]) <= 2e-4, c   # fp32 SIMT path against the fp32 oracle
    assert res["selftest_launch"] == 0
    assert res["status_after_selftest"] == 9      # DF_ERR_DEVICE_BOUNDS, reported once
    assert res["status_again"] == 0
    assert res["status_after_forward"] == 0 and res["finite"]


@pytest.mark.gpu
def test_normal_build_has_no_checker():
    import torch
    from helpers import pkg
    assert torch.cuda.is_available(), "this test needs a GPU"
    p = pkg()
    assert p.lib().df_attn_selftest_bounds_check(None) == p.DF_ERR_UNSUPPORTED
    p.lib().df_attn_last_status()
