"""A layer's worth of this library's stream-aware entry points captured into ONE CUDA graph and replayed: LayerNorm ->
fused Q/K/V projection -> attention forward -> output projection + bias + residual -> GELU, then the backward of GELU,
attention and LayerNorm and a one-launch AdamW step. The reference's own launchers run on the legacy stream, outside
the capturing stream, which is what makes its graph capture fragile (darkforest-cuda/src/lib.rs:259-325 against
kernels/attention_fused.cu:240); every df_* entry point here takes the caller's stream, creates no CUDA object and
allocates nothing, so a capture sees exactly the kernels. Replays must reproduce the eager results: bit for bit where
the kernels are deterministic, to rounding for the LayerNorm column sums (added with atomics)."""
import numpy as np
import pytest

from helpers import pkg

pytestmark = pytest.mark.gpu


def test_layer_forward_backward_and_optimizer_step_replay_from_one_graph(oracle):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    p = pkg()
    B, S, H, D = 2, 512, 12, 64
    d = H * D
    rows = B * S
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    rnd = lambda *shape, s=1.0: torch.randn(shape, device="cuda", generator=g) * s
    x, d_y = rnd(rows, d), rnd(rows, d)
    gamma, beta = 1.0 + rnd(d, s=0.1), rnd(d, s=0.1)
    wq, wk, wv, wo = (rnd(d, d, s=0.02) for _ in range(4))
    bq, bk, bv, bo = (rnd(d, s=0.02) for _ in range(4))
    params0 = [t.clone() for t in (wq, wk, wv, wo)]
    grads = [rnd(d, d, s=0.01) for _ in range(4)]
    moms = [(torch.zeros(d, d, device="cuda"), torch.zeros(d, d, device="cuda")) for _ in range(4)]
    plan = p.AdamwPlan([(w, m, v, gr) for w, (m, v), gr in zip((wq, wk, wv, wo), moms, grads)])
    # every intermediate is allocated up front: nothing is allocated between capture begin and end
    h, q, k, v, a, y, act = (torch.empty(rows, d, device="cuda") for _ in range(7))
    means, rstds = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    lse, delta = torch.empty(B, H, S, device="cuda"), torch.empty(B, H, S, device="cuda")
    d_act, d_q, d_k, d_v, d_x = (torch.empty(rows, d, device="cuda") for _ in range(5))
    d_gamma, d_beta = torch.zeros(d, device="cuda"), torch.zeros(d, device="cuda")
    scale = D ** -0.5
    hyper = (1e-3, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9, 1 - 0.95)

    def layer(stream):
        v3 = lambda t: t.view(B, S, d)
        p.layernorm(x, gamma, beta, out=h, means=means, rstds=rstds, stream=stream)
        p.linear_qkv(h, wq, wk, wv, bq, bk, bv, q=q, k=k, v=v, stream=stream)
        p.forward(v3(q), v3(k), v3(v), H, scale, True, out=v3(a), lse=lse, stream=stream)
        p.linear(a, wo, bo, residual=x, out=y, stream=stream)
        p.gelu(y, out=act, stream=stream)
        p.gelu_backward(d_y, y, grad_x=d_act, stream=stream)
        p.backward(v3(q), v3(k), v3(v), v3(a), v3(d_act), lse, H, scale, True, d_q=v3(d_q), d_k=v3(d_k), d_v=v3(d_v),
                   delta_buf=delta, stream=stream)
        p.layernorm_backward(d_q, x, gamma, means, rstds, grad_x=d_x, grad_gamma=d_gamma, grad_beta=d_beta, stream=stream)
        plan.step(*hyper, stream=stream)

    def reset():
        for w, w0 in zip((wq, wk, wv, wo), params0):
            w.copy_(w0)
        for m, v_ in moms:
            m.zero_()
            v_.zero_()
        d_gamma.zero_()
        d_beta.zero_()

    outputs = (h, q, a, lse, y, act, d_act, d_q, d_k, d_v, d_x, wq, wo, moms[0][0], moms[3][1])
    # eager, on a side stream (also the warm-up every capture needs: kernel attributes, the device status word)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(side)
    side.synchronize()
    assert p.sync_status() == 0
    eager = [t.clone() for t in outputs]
    eager_cols = (d_gamma.clone(), d_beta.clone())
    assert all(bool(torch.isfinite(t).all()) for t in eager)

    reset()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    launches_before = p.launch_count()
    with torch.cuda.graph(graph):
        layer(torch.cuda.current_stream())
    captured = p.launch_count() - launches_before
    assert captured >= 10          # ten calls, at least one kernel each; nothing ran yet:
    torch.cuda.synchronize()
    assert torch.equal(wq, params0[0]) and float(d_gamma.abs().max()) == 0.0
    for _ in range(2):
        reset()
        graph.replay()
        torch.cuda.synchronize()
        assert p.sync_status() == 0
        for got, ref in zip(outputs, eager):
            assert torch.equal(got, ref)
        for got, ref in zip((d_gamma, d_beta), eager_cols):
            assert float((got - ref).abs().max()) <= 1e-4 * max(1.0, float(ref.abs().max()))
    # and the replayed forward is right, not merely repeatable: attention output against the oracle on one sequence
    o_ref, _ = oracle.forward(q.view(B, S, d)[:1].cpu().numpy(), k.view(B, S, d)[:1].cpu().numpy(), v.view(B, S, d)[:1].cpu().numpy(),
                              H, scale, True)
    assert np.abs(a.view(B, S, d)[:1].cpu().numpy() - o_ref).max() <= 2e-3
