"""GPU tests of the ring library (include/darkforest_ring.h), called through its C ABI: single rank on one GPU (all
layouts, fp32 and bf16), the host-side deadline when a peer never arrives, and - where the box has two or more
GPUs - real multi-rank runs over NCCL in child processes (NVLS off: ranks are short-lived test processes)."""
import importlib
import math
import os
import subprocess
import sys
import tempfile
import time

import numpy as np
import pytest

import helpers as hp
from helpers import pkg, rel_err

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _rc():
    pkg().lib()
    return importlib.import_module("dark_forest_b200.ring_c")


@pytest.mark.parametrize("layout", ["contiguous", "zigzag", "balanced"])
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_ring_single_rank_matches_oracle(oracle, layout, dtype):
    """world = 1: no transfer, but the zigzag / balanced layouts still split the sequence into two chunks, so the
    block kernels, the merge, the accumulators, the two compute streams and (balanced) the re-layout copies all run."""
    import torch
    torch.cuda.set_device(0)
    rc = _rc()
    p = pkg()
    bf16 = dtype == "bf16"
    H, S, D = (2, 768, 128) if bf16 else (3, 640, 64)
    scale = 1.0 / math.sqrt(D)
    q, k, v, go = (oracle.fill_normal((1, S, H * D), 321, st) for st in range(4))
    if bf16:
        q, k, v, go = (oracle.round_bf16(x)[0] for x in (q, k, v, go))
    tdt = torch.bfloat16 if bf16 else torch.float32
    tq, tk, tv, tg = (torch.from_numpy(x[0]).cuda().to(tdt) for x in (q, k, v, go))
    ring = rc.Ring(rc.unique_id(), 0, 1, layout, H, S, D, bf16, scale, True, timeout_ms=20000)
    out, lse = torch.empty_like(tq), torch.empty((H, S), device="cuda")
    dq, dk, dv = (torch.empty_like(tq) for _ in range(3))
    ring.forward(tq, tk, tv, out, lse)
    ring.backward(tq, tk, tv, out, tg, lse, dq, dk, dv)
    assert ring.wait() == 0
    assert p.sync_status() == 0
    o_ref, lse_ref = oracle.forward(q, k, v, H, scale, True, f64=bf16)
    g_ref = oracle.backward(q, k, v, go, H, scale, True, f64=bf16)
    tol_o, tol_g = (2e-2, 2e-2) if bf16 else (hp.TOL_O_TF32, hp.TOL_GRAD_REL_TF32)
    assert np.abs(out.float().cpu().numpy() - o_ref[0]).max() <= tol_o
    assert np.abs(lse.cpu().numpy() - lse_ref[0]).max() <= 2e-3
    for got, ref, name in zip((dq, dk, dv), g_ref, ("dq", "dk", "dv")):
        assert rel_err(got.float().cpu().numpy(), ref[0]) <= tol_g, name
    ring.close()


def test_ring_create_gives_up_when_a_peer_never_arrives():
    """A communicator of two ranks of which only this one shows up: the set-up is a host-side rendezvous, so nothing
    runs on the GPU; after the handle's limit the library aborts the communicator and reports DF_ERR_RING_TIMEOUT."""
    import torch
    torch.cuda.set_device(0)
    rc = _rc()
    t0 = time.time()
    with pytest.raises(rc.RingError) as info:
        rc.Ring(rc.unique_id(), 0, 2, "zigzag", 2, 256, 64, False, 0.125, True, timeout_ms=1500)
    assert info.value.status == rc.DF_ERR_RING_TIMEOUT
    assert 1.0 <= time.time() - t0 < 30.0
    # the context is untouched: an ordinary call still works
    p = pkg()
    t = torch.randn((1, 128, 64), device="cuda")
    p.forward(t, t, t, 1, 0.125, True)
    assert p.sync_status() == 0


def _run_ranks(world, layout, dtype, S, H):
    with tempfile.TemporaryDirectory() as tmp:
        id_file = os.path.join(tmp, "ring_id")
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "ring_worker.py"), str(r), str(world), id_file, layout,
                                   dtype, str(S), str(H)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
                 for r in range(world)]
        outs = []
        for pr in procs:
            try:
                o, _ = pr.communicate(timeout=300)
            except subprocess.TimeoutExpired:
                pr.kill()
                o, _ = pr.communicate()
                o += "\n[killed after 300 s]"
            outs.append(o)
        for r, (pr, o) in enumerate(zip(procs, outs)):
            assert pr.returncode == 0 and "RING_WORKER_OK" in o, f"rank {r}:\n{o[-3000:]}"


@pytest.mark.parametrize("layout,dtype", [("zigzag", "fp32"), ("balanced", "fp32"), ("contiguous", "fp32"), ("balanced", "bf16")])
def test_ring_over_nccl_on_all_gpus_of_the_box(layout, dtype):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two or more GPUs")
    world = 2 if n < 4 else 4
    _run_ranks(world, layout, dtype, S=512 * world, H=2)
