"""A static GPT-2 training step around the attention library: the caller side of the hot path.

Follows the op order of the reference's static graph (darkforest-core/src/engine/static_gpt2.rs:
forward 1290-1373, loss head 1386-1418, backward 1440-1574, AdamW 1653-1693) for the full-step
benchmark configuration: per layer LN -> Q,K,V projections -> attention -> output projection +
residual -> LN -> MLP (GELU, tanh form) -> residual; tied LM head + cross-entropy; AdamW
(beta 0.9/0.95, eps 1e-8, weight decay 0.1, static_gpt2.rs:518-521).

This library's code in the step: the attention op, called through the C ABI (df_attn_forward /
df_attn_backward on caller-owned q, k, v, attn_out, lse, delta, d_q, d_k, d_v buffers), and - with
fused_projections - the forward of the projections on either side of it (df_linear_qkv_forward: Q, K, V
in one launch; df_linear_forward: output projection + bias + residual; with step_kernels also
df_linear_gelu_forward: the MLP's first projection with GELU in its epilogue), each inside a
torch.autograd.Function whose backward uses torch matmuls. Everything else (the other cuBLAS TF32
GEMMs, cross-entropy; with step_kernels=False also LayerNorm, GELU and AdamW) is stock torch and stands in for the reference's own
kernels, which are outside the path; the purpose is to measure what share of a step the attention
takes. Weights are N(0, 0.02) from a seed, tokens uniform in [0, vocab).
"""
from __future__ import annotations

import math


def build(pkg, n_layers=12, d_model=768, n_heads=12, d_ff=3072, vocab=50257, max_pos=4096, device="cuda", seed=0,
          fused_projections=True, optimizer=True, step_kernels=True):
    import torch
    import torch.nn as nn
    import torch.nn.functional as F

    timers = {"fwd": [], "bwd": []}

    class Attention(torch.autograd.Function):
        @staticmethod
        def forward(ctx, q, k, v, scale):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            out, lse = pkg.forward(q, k, v, n_heads, scale, True)
            ev1.record()
            timers["fwd"].append((ev0, ev1))
            ctx.save_for_backward(q, k, v, out, lse)
            ctx.scale = scale
            return out

        @staticmethod
        def backward(ctx, d_out):
            q, k, v, out, lse = ctx.saved_tensors
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            d_q, d_k, d_v = pkg.backward(q, k, v, out, d_out.contiguous(), lse, n_heads, ctx.scale, True)
            ev1.record()
            timers["bwd"].append((ev0, ev1))
            return d_q, d_k, d_v, None

    class QKVProjection(torch.autograd.Function):
        """q, k, v = h wq^T + bq, ... in one launch of the library; gradients by torch matmuls."""

        @staticmethod
        def forward(ctx, h, wq, wk, wv, bq, bk, bv):
            q, k, v = pkg.linear_qkv(h, wq, wk, wv, bq, bk, bv)
            ctx.save_for_backward(h, wq, wk, wv)
            return q, k, v

        @staticmethod
        def backward(ctx, dq, dk, dv):
            h, wq, wk, wv = ctx.saved_tensors
            dh = dq @ wq
            dh.addmm_(dk, wk)
            dh.addmm_(dv, wv)
            return dh, dq.t() @ h, dk.t() @ h, dv.t() @ h, dq.sum(0), dk.sum(0), dv.sum(0)

    class OutProjection(torch.autograd.Function):
        """x + a wo^T + bo in one launch (bias and residual added in the GEMM's epilogue)."""

        @staticmethod
        def forward(ctx, a, w, b, res):
            ctx.save_for_backward(a, w)
            return pkg.linear(a, w, b, residual=res)

        @staticmethod
        def backward(ctx, dout):
            a, w = ctx.saved_tensors
            return dout @ w, dout.t() @ a, dout.sum(0), dout

    class LayerNormFn(torch.autograd.Function):
        """This library's LayerNorm (launch_layernorm / launch_layernorm_backward of the reference's step)."""

        @staticmethod
        def forward(ctx, x, gamma, beta):
            x2 = x.reshape(-1, x.shape[-1]).contiguous()
            out, means, rstds = pkg.layernorm(x2, gamma, beta)
            ctx.save_for_backward(x2, gamma, means, rstds)
            return out.view(x.shape)

        @staticmethod
        def backward(ctx, d_out):
            x2, gamma, means, rstds = ctx.saved_tensors
            gg, gb = torch.zeros_like(gamma), torch.zeros_like(gamma)
            gx = pkg.layernorm_backward(d_out.reshape(x2.shape).contiguous(), x2, gamma, means, rstds, grad_gamma=gg, grad_beta=gb)
            return gx.view(d_out.shape), gg, gb

    class GeluFn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            x = x.contiguous()
            ctx.save_for_backward(x)
            return pkg.gelu(x)

        @staticmethod
        def backward(ctx, d_out):
            (x,) = ctx.saved_tensors
            return pkg.gelu_backward(d_out.contiguous(), x)

    class MlpUpFn(torch.autograd.Function):
        """The MLP's first projection with GELU in the projection kernel's epilogue (df_linear_gelu_forward): the
        pre-activation is kept for the backward, which goes through this library's GELU backward and torch matmuls."""

        @staticmethod
        def forward(ctx, x, w, b):
            x2 = x.reshape(-1, x.shape[-1]).contiguous()
            pre, act = pkg.linear_gelu(x2, w, b)
            ctx.save_for_backward(x2, w, pre)
            return act.view(*x.shape[:-1], w.shape[0])

        @staticmethod
        def backward(ctx, d_act):
            x2, w, pre = ctx.saved_tensors
            d_pre = pkg.gelu_backward(d_act.reshape(pre.shape).contiguous(), pre)
            return (d_pre @ w).view(*d_act.shape[:-1], w.shape[1]), d_pre.t() @ x2, d_pre.sum(0)

    class LayerNorm(nn.LayerNorm):
        def forward(self, x):
            return LayerNormFn.apply(x, self.weight, self.bias) if step_kernels else super().forward(x)

    def gelu(x):
        return GeluFn.apply(x) if step_kernels else F.gelu(x, approximate="tanh")

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = LayerNorm(d_model, eps=1e-5), LayerNorm(d_model, eps=1e-5)
            self.wq, self.wk, self.wv, self.wo = (nn.Linear(d_model, d_model) for _ in range(4))
            self.w1, self.w2 = nn.Linear(d_model, d_ff), nn.Linear(d_ff, d_model)

        def forward(self, x):
            h = self.ln1(x)
            scale = (d_model / n_heads) ** -0.5  # static_gpt2.rs:1291
            if fused_projections:
                B, S, _ = x.shape
                q, k, v = QKVProjection.apply(h.reshape(B * S, d_model), self.wq.weight, self.wk.weight, self.wv.weight,
                                              self.wq.bias, self.wk.bias, self.wv.bias)
                a = Attention.apply(q.view(B, S, d_model), k.view(B, S, d_model), v.view(B, S, d_model), scale)
                x = OutProjection.apply(a.reshape(B * S, d_model), self.wo.weight, self.wo.bias,
                                        x.reshape(B * S, d_model).contiguous()).view(B, S, d_model)
            else:
                a = Attention.apply(self.wq(h).contiguous(), self.wk(h).contiguous(), self.wv(h).contiguous(), scale)
                x = x + self.wo(a)
            h2 = self.ln2(x)
            if step_kernels and fused_projections:
                return x + self.w2(MlpUpFn.apply(h2, self.w1.weight, self.w1.bias))
            return x + self.w2(gelu(self.w1(h2)))

    class GPT2(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok, self.pos = nn.Embedding(vocab, d_model), nn.Embedding(max_pos, d_model)
            self.blocks = nn.ModuleList(Block() for _ in range(n_layers))
            self.ln_f = LayerNorm(d_model, eps=1e-5)

        def forward(self, idx, targets):
            B, S = idx.shape
            x = self.tok(idx) + self.pos(torch.arange(S, device=idx.device))[None]
            for blk in self.blocks:
                x = blk(x)
            x = self.ln_f(x)
            # tied LM head + cross-entropy in row chunks, like the reference's chunked loss head
            loss = x.new_zeros(())
            rows = x.reshape(B * S, d_model)
            tgt = targets.reshape(-1)
            chunk = 8192
            for r0 in range(0, B * S, chunk):
                logits = rows[r0:r0 + chunk] @ self.tok.weight.t()
                loss = loss + F.cross_entropy(logits, tgt[r0:r0 + chunk], reduction="sum")
            return loss / (B * S)

    torch.manual_seed(seed)
    torch.backends.cuda.matmul.allow_tf32 = True  # the reference runs its GEMMs in TF32 (lib.rs:47)
    model = GPT2().to(device)
    for name, prm in model.named_parameters():
        if prm.dim() >= 2:
            nn.init.normal_(prm, 0.0, 0.02)
        elif name.endswith("bias"):
            nn.init.zeros_(prm)
    if not optimizer:
        return model, None, timers
    if step_kernels:
        opt = MultiTensorAdamW(pkg, list(model.parameters()), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    return model, opt, timers


class MultiTensorAdamW:
    """AdamW over all parameters in one launch per step (df_adamw_update_multi). Gradients live in buffers allocated
    once, like the reference's persistent gradient tensors (static_gpt2.rs:77-99), so the tensor table is built and
    uploaded once; zero_grad clears them in place."""

    def __init__(self, pkg, params, lr, betas, eps, weight_decay):
        import torch
        self.pkg, self.params = pkg, params
        self.lr, (self.b1, self.b2), self.eps, self.wd, self.t = lr, betas, eps, weight_decay, 0
        for p in params:
            p.grad = torch.zeros_like(p)
        self.m = [torch.zeros_like(p) for p in params]
        self.v = [torch.zeros_like(p) for p in params]
        self.plan = pkg.AdamwPlan([(p.data, m, v, p.grad) for p, m, v in zip(params, self.m, self.v)])

    def zero_grad(self, set_to_none=False):
        import torch
        torch._foreach_zero_([p.grad for p in self.params])

    def step(self):
        self.t += 1
        self.plan.step(self.lr, self.b1, self.b2, self.eps, self.wd, 1.0 - self.b1 ** self.t, 1.0 - self.b2 ** self.t)


def run(pkg, batch=8, seq=4096, steps=3, warmup=1, device="cuda", **model_kw):
    """Returns timing of a full training step and the attention's share of it."""
    import torch
    model, opt, timers = build(pkg, device=device, **model_kw)
    vocab = model.tok.num_embeddings
    gen = torch.Generator(device=device)
    gen.manual_seed(1)
    step_ms, attn_ms, losses = [], [], []
    for it in range(warmup + steps):
        idx = torch.randint(0, vocab, (batch, seq), device=device, generator=gen)
        tgt = torch.randint(0, vocab, (batch, seq), device=device, generator=gen)
        timers["fwd"].clear()
        timers["bwd"].clear()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loss = model(idx, tgt)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        e1.record()
        torch.cuda.synchronize()
        if it >= warmup:
            step_ms.append(e0.elapsed_time(e1))
            attn_ms.append((sum(a.elapsed_time(b) for a, b in timers["fwd"]), sum(a.elapsed_time(b) for a, b in timers["bwd"])))
            losses.append(float(loss))
    n = len(step_ms)
    fwd = sum(a for a, _ in attn_ms) / n
    bwd = sum(b for _, b in attn_ms) / n
    step = sum(step_ms) / n
    return {"step_ms": step, "attention_fwd_ms": fwd, "attention_bwd_ms": bwd, "attention_share": (fwd + bwd) / step,
            "tokens_per_s": batch * seq / (step * 1e-3), "loss_first_step": losses[0], "ln_vocab": math.log(vocab),
            "batch": batch, "seq": seq}
