"""Generates tests/golden/attention_golden.npz and tests/golden/step_golden.npz (see main_step).

Expected values come from an implementation that is independent of the oracle under
test: torch's CPU scaled_dot_product_attention in float64 plus autograd, which is the
twin the reference itself checks its attention against (scripts/verify_loss_parity.py:58).

Cases
  kat_fwd   the reference's forward known-answer test, darkforest-cuda/src/lib.rs:2606-2628
            (single head, S=5, D=4, q=(i-7)/11, k=(3-i)/13, v=sin(i), scale 1/2, causal)
  kat_bwd   the reference's backward known-answer test, lib.rs:2753-2769
            (single head, S=4, D=3, q=(i-4)/9, k=(2-i)/10, v=(i+1)/8, dO=(i-3)/7, scale 1/sqrt 3)
  mh_*      seeded multi-head cases (inputs from the oracle's counter-based generator,
            seed and stream stored), including ragged S and the CPU-runnable benchmark
            configuration B=1,H=12,S=128,D=64 stored on a row sample.
  dec_*     seeded one-token decode cases over a KV cache (attention_fused.cu:551-615): expected
            output and logsumexp per head.

Run:  python tests/golden/make_golden.py     (CPU only; needs torch and the built oracle)
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle.attn_oracle import Oracle  # noqa: E402  (input generator only)


def torch_expected(q, k, v, d_out, H, scale, causal):
    """q,k,v,d_out: [B,S,H*D] float32 numpy -> dict of float64 numpy."""
    B, S, dm = q.shape
    D = dm // H

    def heads(x):
        return torch.tensor(x, dtype=torch.float64).reshape(B, S, H, D).transpose(1, 2).clone().requires_grad_(True)

    qh, kh, vh = heads(q), heads(k), heads(v)
    out = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale)
    go = torch.tensor(d_out, dtype=torch.float64).reshape(B, S, H, D).transpose(1, 2)
    (out * go).sum().backward()
    s = (qh.detach() @ kh.detach().transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(~torch.tril(torch.ones(S, S, dtype=torch.bool)), -math.inf)
    lse = torch.logsumexp(s, -1)

    def flat(x):
        return x.detach().transpose(1, 2).reshape(B, S, dm).numpy()

    return dict(out=flat(out), lse=lse.numpy(), dq=flat(qh.grad), dk=flat(kh.grad), dv=flat(vh.grad))


def main():
    orc = Oracle()
    store = {}

    # --- reference known-answer tests (closed-form inputs) ---
    n = 5 * 4
    i = np.arange(n, dtype=np.float32)
    q = ((i - 7.0) / 11.0).astype(np.float32).reshape(1, 5, 4)
    k = ((3.0 - i) / 13.0).astype(np.float32).reshape(1, 5, 4)
    v = np.sin(i).astype(np.float32).reshape(1, 5, 4)
    go = np.ones_like(q)
    e = torch_expected(q, k, v, go, 1, 1.0 / math.sqrt(4.0), True)
    store.update({"kat_fwd_q": q, "kat_fwd_k": k, "kat_fwd_v": v, "kat_fwd_out": e["out"], "kat_fwd_lse": e["lse"]})

    n = 4 * 3
    i = np.arange(n, dtype=np.float32)
    q = ((i - 4.0) / 9.0).astype(np.float32).reshape(1, 4, 3)
    k = ((2.0 - i) / 10.0).astype(np.float32).reshape(1, 4, 3)
    v = ((i + 1.0) / 8.0).astype(np.float32).reshape(1, 4, 3)
    go = ((i - 3.0) / 7.0).astype(np.float32).reshape(1, 4, 3)
    e = torch_expected(q, k, v, go, 1, 1.0 / math.sqrt(3.0), True)
    store.update({"kat_bwd_q": q, "kat_bwd_k": k, "kat_bwd_v": v, "kat_bwd_do": go})
    store.update({f"kat_bwd_{n}": e[n] for n in ("out", "lse", "dq", "dk", "dv")})

    # --- seeded multi-head cases: name -> (B,H,S,D,causal,seed) ---
    cases = {
        "mh_small": (2, 3, 17, 8, True, 0xDF10),
        "mh_noncausal": (1, 2, 33, 16, False, 0xDF11),
        "mh_d128": (1, 2, 40, 128, True, 0xDF12),
        "mh_ragged": (1, 2, 129, 64, True, 0xDF13),
        "mh_cfg1": (1, 12, 128, 64, True, 0xDF01),
    }
    meta = []
    for name, (B, H, S, D, causal, seed) in cases.items():
        shape = (B, S, H * D)
        q, k, v, go = (orc.fill_normal(shape, seed, st) for st in range(4))
        e = torch_expected(q, k, v, go, H, 1.0 / math.sqrt(D), causal)
        rows = np.arange(S) if S <= 40 else np.unique(np.r_[0:3, S // 2 - 1:S // 2 + 1, S - 3:S])
        store[f"{name}_rows"] = rows.astype(np.int64)
        for n in ("out", "dq", "dk", "dv"):
            store[f"{name}_{n}"] = e[n][:, rows, :]
        store[f"{name}_lse"] = e["lse"][:, :, rows]
        meta.append((name, B, H, S, D, int(causal), seed))
    store["cases"] = np.array([m[0] for m in meta])
    store["case_params"] = np.array([m[1:] for m in meta], dtype=np.int64)

    # --- decode cases: one query token over T cached tokens; name -> (H, D, T, T_max, seed) ---
    # expected = softmax(scale * q K^T) V in float64 with torch (independent of the oracle)
    dec_cases = {"dec_small": (4, 64, 37, 64, 0xDF20), "dec_d128": (2, 128, 300, 320, 0xDF21),
                 "dec_odd": (3, 33, 129, 160, 0xDF22), "dec_cfg": (12, 64, 1000, 1024, 0xDF23)}
    dmeta = []
    for name, (H, D, T, T_max, seed) in dec_cases.items():
        q = orc.fill_normal((H * D,), seed, 0)
        k, v = (orc.fill_normal((T_max, H * D), seed, st) for st in (1, 2))
        qh = torch.tensor(q, dtype=torch.float64).reshape(H, 1, D)
        kh = torch.tensor(k[:T], dtype=torch.float64).reshape(T, H, D).transpose(0, 1)
        vh = torch.tensor(v[:T], dtype=torch.float64).reshape(T, H, D).transpose(0, 1)
        sc = (qh @ kh.transpose(-1, -2)) / math.sqrt(D)
        store[f"{name}_out"] = (torch.softmax(sc, -1) @ vh).reshape(H * D).numpy()
        store[f"{name}_lse"] = torch.logsumexp(sc, -1).reshape(H).numpy()
        dmeta.append((name, H, D, T, T_max, seed))
    store["dec_cases"] = np.array([m[0] for m in dmeta])
    store["dec_case_params"] = np.array([m[1:] for m in dmeta], dtype=np.int64)

    # --- linear projection: out = x w^T + b (+ residual) in float64 with torch (independent of the oracle) ---
    lin_cases = {"lin_small": (37, 48, 20, 0xDF30), "lin_gpt2_rows": (96, 768, 768, 0xDF31)}
    lmeta = []
    for name, (rows, fin, fout, seed) in lin_cases.items():
        x = orc.fill_normal((rows, fin), seed, 0)
        w = (orc.fill_normal((fout, fin), seed, 1) * 0.02).astype(np.float32)
        b = (orc.fill_normal((fout,), seed, 2) * 0.02).astype(np.float32)
        r = orc.fill_normal((rows, fout), seed, 3)
        t64 = lambda a: torch.tensor(a, dtype=torch.float64)
        y = t64(x) @ t64(w).t() + t64(b)
        store[f"{name}_out"] = y.numpy()
        store[f"{name}_out_res"] = (y + t64(r)).numpy()
        lmeta.append((name, rows, fin, fout, seed))
    store["lin_cases"] = np.array([m[0] for m in lmeta])
    store["lin_case_params"] = np.array([m[1:] for m in lmeta], dtype=np.int64)

    # --- loss head: log-softmax cross-entropy of a chunk in float64 with torch (independent of the oracle) ---
    ce_cases = {"ce_small": (7, 33, 16, 0xDF40), "ce_vocab_row": (3, 50257, 512, 0xDF41)}
    cmeta = []
    for name, (rows, cols, total_rows, seed) in ce_cases.items():
        z = (orc.fill_normal((rows, cols), seed, 0) * 3.0).astype(np.float32)
        tg = (np.abs(orc.fill_normal((rows,), seed, 1)) * 1000003).astype(np.int64) % cols
        z64 = torch.tensor(z, dtype=torch.float64)
        lp = torch.log_softmax(z64, -1)
        store[f"{name}_loss"] = np.array(float(-lp[torch.arange(rows), torch.tensor(tg)].sum() / total_rows))
        p = torch.softmax(z64, -1)
        gsel = p.clone()
        gsel[torch.arange(rows), torch.tensor(tg)] -= 1.0
        cols_keep = np.unique(np.r_[0:8, cols - 8:cols, tg])
        store[f"{name}_cols"] = cols_keep.astype(np.int64)
        store[f"{name}_probs"] = p[:, cols_keep].numpy()
        store[f"{name}_grad"] = (gsel / total_rows)[:, cols_keep].numpy()
        store[f"{name}_targets"] = tg.astype(np.int64)
        cmeta.append((name, rows, cols, total_rows, seed))
    store["ce_cases"] = np.array([m[0] for m in cmeta])
    store["ce_case_params"] = np.array([m[1:] for m in cmeta], dtype=np.int64)

    path = os.path.join(HERE, "attention_golden.npz")
    np.savez_compressed(path, **store)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_step():
    """tests/golden/step_golden.npz: LayerNorm forward / backward, tanh-GELU forward / backward and two AdamW steps,
    computed by torch on the CPU in float64 (torch.nn.functional.layer_norm and gelu with autograd; AdamW written out
    from its definition, the form the reference's own test uses, darkforest-cuda/src/lib.rs:2721-2751). Inputs come
    from the oracle's counter-based generator (seed and stream stored)."""
    orc = Oracle()
    store = {}
    ln_cases = {"ln_small": (5, 12, 0xDF50), "ln_ragged": (7, 50, 0xDF51), "ln_model": (9, 768, 0xDF52), "ln_wide": (2, 1600, 0xDF53)}
    meta = []
    for name, (rows, cols, seed) in ln_cases.items():
        x = (orc.fill_normal((rows, cols), seed, 0) * 1.7 + 0.3).astype(np.float32)
        gamma = (1.0 + 0.2 * orc.fill_normal((cols,), seed, 1)).astype(np.float32)
        beta = (0.1 * orc.fill_normal((cols,), seed, 2)).astype(np.float32)
        go = orc.fill_normal((rows, cols), seed, 3).astype(np.float32)
        xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
        gt = torch.tensor(gamma, dtype=torch.float64, requires_grad=True)
        bt = torch.tensor(beta, dtype=torch.float64, requires_grad=True)
        out = torch.nn.functional.layer_norm(xt, (cols,), gt, bt, eps=1e-5)
        out.backward(torch.tensor(go, dtype=torch.float64))
        store[f"{name}_out"] = out.detach().numpy()
        store[f"{name}_mean"] = xt.detach().mean(1).numpy()
        store[f"{name}_rstd"] = (1.0 / torch.sqrt(xt.detach().var(1, unbiased=False) + 1e-5)).numpy()
        store[f"{name}_gx"] = xt.grad.numpy()
        store[f"{name}_ggamma"] = gt.grad.numpy()
        store[f"{name}_gbeta"] = bt.grad.numpy()
        meta.append((name, rows, cols, seed))
    store["ln_cases"] = np.array([m[0] for m in meta])
    store["ln_case_params"] = np.array([m[1:] for m in meta], dtype=np.int64)

    n, seed = 4099, 0xDF54
    x = (orc.fill_normal((n,), seed, 0) * 2.5).astype(np.float32)
    x[:5] = [-2.0, -1.0, 0.0, 1.0, 2.0]   # the reference's own test points, lib.rs:2832-2848
    go = orc.fill_normal((n,), seed, 1).astype(np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    y = torch.nn.functional.gelu(xt, approximate="tanh")
    y.backward(torch.tensor(go, dtype=torch.float64))
    store["gelu_params"] = np.array([n, seed], dtype=np.int64)
    store["gelu_out"] = y.detach().numpy()
    store["gelu_gx"] = xt.grad.numpy()

    n, seed = 1003, 0xDF55
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    p = orc.fill_normal((n,), seed, 0).astype(np.float64)
    m = np.zeros(n)
    v = np.zeros(n)
    for t in (1, 2):
        g = orc.fill_normal((n,), seed, t).astype(np.float64)
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        p = p * (1 - lr * wd) - lr * (m / (1 - b1 ** t)) / (np.sqrt(v / (1 - b2 ** t)) + eps)
        store[f"adamw_p{t}"], store[f"adamw_m{t}"], store[f"adamw_v{t}"] = p.copy(), m.copy(), v.copy()
    store["adamw_params"] = np.array([n, seed], dtype=np.int64)
    store["adamw_hyper"] = np.array([lr, b1, b2, eps, wd])

    path = os.path.join(HERE, "step_golden.npz")
    np.savez_compressed(path, **store)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    # `python tests/golden/make_golden.py step` writes step_golden.npz only
    if "step" not in sys.argv[1:]:
        main()
    main_step()
