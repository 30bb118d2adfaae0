"""The reference's StaticGPT2 checkpoint file (darkforest-core/src/engine/static_gpt2.rs:1924-2114): the Python and the
C++ implementations against a byte image built here straight from the format's description, and against each other.
Host-only: no GPU involved."""
import importlib
import os
import struct
import subprocess

import numpy as np
import pytest

from helpers import pkg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOOL = os.path.join(ROOT, "dark-forest_b200", "lib", "checkpoint_tool")


def _ck():
    pkg()
    return importlib.import_module("dark_forest_b200.checkpoint")


def _tiny(ck):
    cfg = ck.GPT2Config(vocab_size=11, d_model=8, n_heads=2, n_layers=2, d_ff=12, seq_len=5)
    rng = np.random.default_rng(7)
    w = {n: rng.standard_normal(cfg.shape_of(n)).astype(np.float32) for n in cfg.tensor_names()}
    m = {n: (rng.standard_normal(cfg.shape_of(n)).astype(np.float32), rng.random(cfg.shape_of(n)).astype(np.float32))
         for n in cfg.tensor_names()}
    return cfg, ck.Checkpoint(w, m, step_count=1234, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)


def _image_from_the_format(cfg, c):
    """The file as save_checkpoint's source describes it, written without the code under test."""
    order = ["tok_emb", "pos_emb", "ln_f_gamma", "ln_f_beta", "lm_head"]
    per_layer = ["ln1_gamma", "ln1_beta", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "ln2_gamma", "ln2_beta", "w1", "b1",
                 "w2", "b2"]
    for l in range(cfg.n_layers):
        order += [f"layers.{l}.{n}" for n in per_layer]
    out = b""
    for n in order:
        a = c.weights[n].astype("<f4").ravel()
        out += struct.pack("<Q", a.size) + a.tobytes()
    for n in order:
        for a in c.moments[n]:
            a = a.astype("<f4").ravel()
            out += struct.pack("<Q", a.size) + a.tobytes()
    out += struct.pack("<Q", c.step_count) + struct.pack("<5f", c.lr, c.beta1, c.beta2, c.eps, c.wd)
    return out


def test_python_writer_matches_the_format_and_reads_back(tmp_path):
    ck = _ck()
    cfg, c = _tiny(ck)
    path = str(tmp_path / "tiny.ckpt")
    ck.save_checkpoint(path, cfg, c)
    raw = open(path, "rb").read()
    assert raw == _image_from_the_format(cfg, c)
    assert len(raw) == ck.expected_file_bytes(cfg)
    back = ck.load_checkpoint(path, cfg)
    assert back.step_count == 1234 and back.lr == np.float32(1e-3) and back.wd == np.float32(0.1)
    for n in cfg.tensor_names():
        assert np.array_equal(back.weights[n], c.weights[n]) and back.weights[n].shape == cfg.shape_of(n)
        assert np.array_equal(back.moments[n][0], c.moments[n][0]) and np.array_equal(back.moments[n][1], c.moments[n][1])


def test_loader_rejects_another_configuration_with_the_reference_message(tmp_path):
    ck = _ck()
    cfg, c = _tiny(ck)
    path = str(tmp_path / "tiny.ckpt")
    ck.save_checkpoint(path, cfg, c)
    other = ck.GPT2Config(vocab_size=11, d_model=8, n_heads=2, n_layers=2, d_ff=12, seq_len=6)
    with pytest.raises(ck.CheckpointError, match=r"tensor size mismatch: file=40 model=48"):
        ck.load_checkpoint(path, other)
    open(path, "wb").write(open(path, "rb").read()[:-3])
    with pytest.raises(ck.CheckpointError, match="failed to fill whole buffer"):
        ck.load_checkpoint(path, cfg)


def test_cpp_reader_and_writer_round_trip_the_same_bytes(tmp_path):
    ck = _ck()
    cfg, c = _tiny(ck)
    src, dst = str(tmp_path / "a.ckpt"), str(tmp_path / "b.ckpt")
    ck.save_checkpoint(src, cfg, c)
    args = [str(x) for x in (cfg.vocab_size, cfg.d_model, cfg.n_heads, cfg.n_layers, cfg.d_ff, cfg.seq_len)]
    if not os.path.exists(TOOL):
        subprocess.run(["make", "-C", os.path.join(ROOT, "dark-forest_b200", "host")], check=True, capture_output=True)
    r = subprocess.run([TOOL, src, dst] + args, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert open(dst, "rb").read() == open(src, "rb").read()
    assert '"step_count": 1234' in r.stdout and '"tensors": 37' in r.stdout
    bad = subprocess.run([TOOL, src, dst, "11", "8", "2", "2", "12", "6"], capture_output=True, text=True)
    assert bad.returncode == 1 and "tensor size mismatch: file=40 model=48" in bad.stderr


def test_harness_weights_go_through_the_reference_format(tmp_path):
    """The GPT-2 step harness's weights written in the reference's format and loaded into a second model (CPU):
    same parameters afterwards; the tied LM head is written to both of the reference's blocks."""
    import torch
    ck = _ck()
    step = importlib.import_module("dark_forest_b200.gpt2_step")
    kw = dict(n_layers=2, d_model=16, n_heads=2, d_ff=32, vocab=23, max_pos=9, device="cpu")
    model_a, _, _ = step.build(None, seed=1, optimizer=False, **kw)
    model_b, _, _ = step.build(None, seed=2, optimizer=False, **kw)
    cfg = ck.GPT2Config(vocab_size=23, d_model=16, n_heads=2, n_layers=2, d_ff=32, seq_len=9)
    path = str(tmp_path / "harness.ckpt")
    ck.save_checkpoint(path, cfg, ck.from_torch_model(model_a, None, cfg, step_count=5))
    assert os.path.getsize(path) == ck.expected_file_bytes(cfg)
    loaded = ck.load_checkpoint(path, cfg)
    assert loaded.step_count == 5 and np.array_equal(loaded.weights["lm_head"], loaded.weights["tok_emb"])
    ck.into_torch_model(loaded, model_b)
    for (na, pa), (nb, pb) in zip(model_a.named_parameters(), model_b.named_parameters()):
        assert na == nb and torch.equal(pa, pb), na
