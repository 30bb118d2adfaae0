"""The reference's StaticGPT2 checkpoint file, read and written bit for bit
(darkforest-core/src/engine/static_gpt2.rs:1924-2006 save_checkpoint, :2012-2114 load_checkpoint).

Format (all little endian): one block per tensor, `u64 element count` followed by that many `f32`; first the weights -
tok_emb [vocab, d], pos_emb [seq, d], ln_f_gamma [d], ln_f_beta [d], lm_head [vocab, d], then per layer ln1_gamma,
ln1_beta, wq, bq, wk, bk, wv, bv, wo, bo, ln2_gamma, ln2_beta, w1 [d_ff, d], b1 [d_ff], w2 [d, d_ff], b2 - then the
AdamW moments in the same order, two blocks (m, v) per tensor; then a footer `u64 step_count` and five `f32`: lr,
beta1, beta2, eps, wd. The file carries no shapes and no hyper-parameters: the reader must know the model's
configuration and fails with the reference's message ("load_checkpoint: tensor size mismatch: file=.. model=..")
when a block's length differs. Host-side code only (numpy); it is how weights move between this repository's GPT-2
step harness and the reference.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import numpy as np

GLOBAL_TENSORS = ("tok_emb", "pos_emb", "ln_f_gamma", "ln_f_beta", "lm_head")
LAYER_TENSORS = ("ln1_gamma", "ln1_beta", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "ln2_gamma", "ln2_beta",
                 "w1", "b1", "w2", "b2")


@dataclass(frozen=True)
class GPT2Config:
    vocab_size: int
    d_model: int
    n_heads: int
    n_layers: int
    d_ff: int
    seq_len: int

    def shape_of(self, name: str) -> Tuple[int, ...]:
        base = name.split(".")[-1]
        d, f = self.d_model, self.d_ff
        return {"tok_emb": (self.vocab_size, d), "pos_emb": (self.seq_len, d), "lm_head": (self.vocab_size, d),
                "ln_f_gamma": (d,), "ln_f_beta": (d,), "ln1_gamma": (d,), "ln1_beta": (d,), "ln2_gamma": (d,), "ln2_beta": (d,),
                "wq": (d, d), "wk": (d, d), "wv": (d, d), "wo": (d, d), "bq": (d,), "bk": (d,), "bv": (d,), "bo": (d,),
                "w1": (f, d), "b1": (f,), "w2": (d, f), "b2": (d,)}[base]

    def tensor_names(self) -> List[str]:
        """Weight tensors in file order; per-layer names are 'layers.<l>.<name>'."""
        return list(GLOBAL_TENSORS) + [f"layers.{l}.{n}" for l in range(self.n_layers) for n in LAYER_TENSORS]


@dataclass
class Checkpoint:
    weights: Dict[str, np.ndarray]
    moments: Dict[str, Tuple[np.ndarray, np.ndarray]]  # name -> (m, v)
    step_count: int = 0
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    wd: float = 0.1
    extra: dict = field(default_factory=dict)


class CheckpointError(ValueError):
    pass


def _block(a: np.ndarray) -> bytes:
    a = np.ascontiguousarray(a, dtype="<f4")
    return struct.pack("<Q", a.size) + a.tobytes()


def save_checkpoint(path: str, cfg: GPT2Config, ck: Checkpoint) -> None:
    names = cfg.tensor_names()
    with open(path, "wb") as f:
        for n in names:
            w = ck.weights[n]
            if tuple(w.shape) != cfg.shape_of(n):
                raise CheckpointError(f"save_checkpoint: {n} has shape {tuple(w.shape)}, the configuration says {cfg.shape_of(n)}")
            f.write(_block(w))
        for n in names:
            m, v = ck.moments[n]
            if m.size != ck.weights[n].size or v.size != ck.weights[n].size:
                raise CheckpointError(f"save_checkpoint: moments of {n} do not match its size")
            f.write(_block(m))
            f.write(_block(v))
        f.write(struct.pack("<Qfffff", int(ck.step_count), ck.lr, ck.beta1, ck.beta2, ck.eps, ck.wd))


def load_checkpoint(path: str, cfg: GPT2Config) -> Checkpoint:
    names = cfg.tensor_names()
    with open(path, "rb") as f:
        def read_block(name):
            head = f.read(8)
            if len(head) != 8:
                raise CheckpointError("load_checkpoint: failed to fill whole buffer")  # read_exact's message
            (n,) = struct.unpack("<Q", head)
            want = int(np.prod(cfg.shape_of(name)))
            if n != want:
                raise CheckpointError(f"load_checkpoint: tensor size mismatch: file={n} model={want}")
            raw = f.read(4 * n)
            if len(raw) != 4 * n:
                raise CheckpointError("load_checkpoint: failed to fill whole buffer")
            return np.frombuffer(raw, dtype="<f4").astype(np.float32).reshape(cfg.shape_of(name))

        weights = {n: read_block(n) for n in names}
        moments = {}
        for n in names:
            m = read_block(n)
            v = read_block(n)
            moments[n] = (m, v)
        foot = f.read(28)
        if len(foot) != 28:
            raise CheckpointError("load_checkpoint: failed to fill whole buffer")
        step, lr, b1, b2, eps, wd = struct.unpack("<Qfffff", foot)
        return Checkpoint(weights, moments, int(step), lr, b1, b2, eps, wd)


def expected_file_bytes(cfg: GPT2Config) -> int:
    n = sum(int(np.prod(cfg.shape_of(t))) for t in cfg.tensor_names())
    blocks = len(cfg.tensor_names())
    return 3 * (8 * blocks + 4 * n) + 28


# ---- the GPT-2 step harness of this package <-> the reference's tensor names -------------------------------------------
def from_torch_model(model, opt, cfg: GPT2Config, step_count: int = 0) -> Checkpoint:
    """Checkpoint of dark-forest_b200/gpt2_step.py's model. That model ties the LM head to the token embedding (the
    reference keeps a separate lm_head tensor, static_gpt2.rs:299): the embedding is written to both blocks."""
    def arr(t):
        return t.detach().float().cpu().numpy()

    def mom(p):
        st = opt.state.get(p, {}) if opt is not None else {}
        if "exp_avg" in st:
            return arr(st["exp_avg"]), arr(st["exp_avg_sq"])
        z = np.zeros(tuple(p.shape), np.float32)
        return z, z.copy()

    w, m = {}, {}

    def put(name, p):
        w[name] = arr(p)
        m[name] = mom(p)

    put("tok_emb", model.tok.weight)
    put("pos_emb", model.pos.weight)
    put("ln_f_gamma", model.ln_f.weight)
    put("ln_f_beta", model.ln_f.bias)
    put("lm_head", model.tok.weight)
    for l, blk in enumerate(model.blocks):
        pre = f"layers.{l}."
        for name, p in (("ln1_gamma", blk.ln1.weight), ("ln1_beta", blk.ln1.bias), ("wq", blk.wq.weight), ("bq", blk.wq.bias),
                        ("wk", blk.wk.weight), ("bk", blk.wk.bias), ("wv", blk.wv.weight), ("bv", blk.wv.bias),
                        ("wo", blk.wo.weight), ("bo", blk.wo.bias), ("ln2_gamma", blk.ln2.weight), ("ln2_beta", blk.ln2.bias),
                        ("w1", blk.w1.weight), ("b1", blk.w1.bias), ("w2", blk.w2.weight), ("b2", blk.w2.bias)):
            put(pre + name, p)
    g = opt.param_groups[0] if opt is not None else {}
    b1, b2 = g.get("betas", (0.9, 0.95))
    return Checkpoint(w, m, step_count, float(g.get("lr", 3e-4)), float(b1), float(b2), float(g.get("eps", 1e-8)),
                      float(g.get("weight_decay", 0.1)))


def into_torch_model(ck: Checkpoint, model) -> None:
    """Loads the weights of a checkpoint into gpt2_step.py's model (lm_head must equal tok_emb there: tied)."""
    import torch
    if not np.array_equal(ck.weights["lm_head"], ck.weights["tok_emb"]):
        raise CheckpointError("this harness ties the LM head to the token embedding; the checkpoint's lm_head differs")

    def put(p, name):
        with torch.no_grad():
            p.copy_(torch.from_numpy(np.ascontiguousarray(ck.weights[name])).to(p.device))

    put(model.tok.weight, "tok_emb")
    put(model.pos.weight, "pos_emb")
    put(model.ln_f.weight, "ln_f_gamma")
    put(model.ln_f.bias, "ln_f_beta")
    for l, blk in enumerate(model.blocks):
        pre = f"layers.{l}."
        for name, p in (("ln1_gamma", blk.ln1.weight), ("ln1_beta", blk.ln1.bias), ("wq", blk.wq.weight), ("bq", blk.wq.bias),
                        ("wk", blk.wk.weight), ("bk", blk.wk.bias), ("wv", blk.wv.weight), ("bv", blk.wv.bias),
                        ("wo", blk.wo.weight), ("bo", blk.wo.bias), ("ln2_gamma", blk.ln2.weight), ("ln2_beta", blk.ln2.bias),
                        ("w1", blk.w1.weight), ("b1", blk.w1.bias), ("w2", blk.w2.weight), ("b2", blk.w2.bias)):
            put(p, pre + name)
