"""The C++ host layer (dark-forest_b200/host): built binaries exist (CPU check) and the self-test,
which restates the reference's two GPU unit tests through AttentionContext, passes on a GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "dark-forest_b200", "lib")


def test_host_binaries_are_built():
    if not os.path.exists(os.path.join(LIB, "host_selftest")):
        subprocess.run(["make", "-C", os.path.join(ROOT, "dark-forest_b200"), "-j8"], check=True, capture_output=True)
        subprocess.run(["make", "-C", os.path.join(ROOT, "dark-forest_b200", "host"), "-j8"], check=True, capture_output=True)
    for name in ("host_selftest", "bench_sequence_limit", "libdarkforest_kernels.a", "libdarkforest_kernels.so"):
        assert os.path.exists(os.path.join(LIB, name)), name


@pytest.mark.gpu
def test_cpp_host_selftest_passes_on_gpu():
    r = subprocess.run([os.path.join(LIB, "host_selftest")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("ok  ") >= 5 and "FAIL" not in r.stdout


@pytest.mark.gpu
def test_cpp_bench_sequence_limit_small_sweep(tmp_path):
    out = tmp_path / "scaling.json"
    r = subprocess.run([os.path.join(LIB, "bench_sequence_limit"), "--max-seq", "16384", "--random", "--out", str(out)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    import json
    data = json.loads(out.read_text())
    assert [x["seq_len"] for x in data["results"]] == [8192, 16384]
    assert all(x["latency_ms"] > 0 and x["tflops"] > 1.0 for x in data["results"])
    assert data["metadata"]["heads"] == 12 and data["metadata"]["d_head"] == 64
