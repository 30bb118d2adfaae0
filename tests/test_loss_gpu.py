"""GPU parity of the loss head's fused softmax + cross-entropy (launch_fused_chunked_logit_ce, launch_chunked_ce_eval and
df_chunked_logit_ce), through the C ABI, against the CPU oracle, the float64 golden vectors and the reference's own
kernels compiled unmodified. fp32 arithmetic like the reference (its __expf / __logf): probabilities to 2e-5 relative
(+ 1e-7 absolute; __expf's error grows with the distance from the row maximum), gradients likewise (they are the
probabilities divided by the row count), the loss to 1e-5 relative (it is summed in a different order everywhere)."""
import numpy as np
import pytest

from helpers import pkg, to_dev

pytestmark = pytest.mark.gpu


def _close(got, ref, scale=1.0):
    """|got - ref| <= (1e-7 + 2e-5 |ref|) * scale, elementwise; returns the worst ratio (<= 1 passes)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float((np.abs(got - ref) / ((1e-7 + 2e-5 * np.abs(ref)) * scale)).max())


def _case(oracle, rows, cols, seed, spread=3.0):
    z = (oracle.fill_normal((rows, cols), seed, 0) * spread).astype(np.float32)
    tg = ((np.abs(oracle.fill_normal((rows,), seed, 1)) * 1000003).astype(np.int64) % cols).astype(np.int32)
    return z, tg


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (5, 33), (64, 1000), (9, 4097), (150, 50257), (512, 50257), (4, 60001)])
def test_chunked_cross_entropy_matches_oracle(oracle, rows, cols, variant):
    """Vocabulary sizes that leave rows at every 16-byte phase (odd cols), a row longer than shared memory (60001), more
    rows than SMs, and the full chunk of the static step (512 x 50257)."""
    import torch
    torch.cuda.set_device(0)
    p = pkg()
    prev_variant = p.set_option(p.OPT_CE_VARIANT, variant)  # 1: row resident in shared memory, 2: second pass out of L2
    z, tg = _case(oracle, rows, cols, 600 + rows + cols)
    total = max(rows, 512)
    tz, tt = to_dev(z, tg)
    grad = torch.empty_like(tz)
    loss = torch.full((1,), 0.25, device="cuda")           # accumulates on top of what is there
    p.chunked_logit_ce(tz, tt, loss, total, grad_logits=grad)
    assert p.sync_status() == 0
    probs_ref, grad_ref, loss_ref = oracle.chunked_ce(z, tg, total, train=True)
    assert _close(tz.cpu().numpy(), probs_ref) <= 1.0
    assert np.abs(grad.cpu().numpy() - grad_ref).max() <= 3e-5 / total + 1e-9
    assert abs(float(loss) - 0.25 - loss_ref) <= 1e-5 * max(1.0, abs(loss_ref))
    # eval form: logits untouched, same loss
    tz2 = to_dev(z)[0]
    loss2 = torch.zeros(1, device="cuda")
    p.chunked_logit_ce(tz2, tt, loss2, total)
    assert p.sync_status() == 0
    assert torch.equal(tz2, to_dev(z)[0])
    assert abs(float(loss2) - loss_ref) <= 1e-5 * max(1.0, abs(loss_ref))
    p.set_option(p.OPT_CE_VARIANT, prev_variant)


def test_chunked_cross_entropy_golden_and_legacy_symbols(oracle, golden):
    import torch
    torch.cuda.set_device(0)
    p = pkg()
    L = p.lib()
    for name, (rows, cols, total_rows, seed) in zip(golden["ce_cases"], golden["ce_case_params"]):
        z = (oracle.fill_normal((int(rows), int(cols)), int(seed), 0) * 3.0).astype(np.float32)
        tg = golden[f"{name}_targets"].astype(np.int32)
        keep = golden[f"{name}_cols"]
        tz, tt = to_dev(z, tg)
        grad, loss = torch.empty_like(tz), torch.zeros(1, device="cuda")
        torch.cuda.synchronize()
        L.launch_fused_chunked_logit_ce(tz.data_ptr(), tt.data_ptr(), grad.data_ptr(), loss.data_ptr(), int(rows), int(cols),
                                        int(total_rows))
        assert p.sync_status() == 0
        want = float(golden[f"{name}_loss"])
        assert abs(float(loss) - want) <= 1e-5 * max(1.0, abs(want)), name
        assert _close(tz.cpu().numpy()[:, keep], golden[f"{name}_probs"]) <= 1.0, name
        assert np.abs(grad.cpu().numpy()[:, keep] - golden[f"{name}_grad"]).max() <= 3e-5 / int(total_rows) + 1e-9, name
        tz2, loss2 = to_dev(z)[0], torch.zeros(1, device="cuda")
        L.launch_chunked_ce_eval(tz2.data_ptr(), tt.data_ptr(), loss2.data_ptr(), int(rows), int(cols), int(total_rows))
        assert p.sync_status() == 0
        assert abs(float(loss2) - want) <= 1e-5 * max(1.0, abs(want)), name


def test_chunked_cross_entropy_matches_reference_cuda_kernels(oracle):
    """The reference's own softmax.cu, compiled unmodified into oracle/_ref, on the same chunk."""
    import os
    import torch
    from oracle.attn_oracle import REFERENCE_SO, ReferenceKernels
    if not os.path.exists(REFERENCE_SO):
        pytest.skip("oracle/_ref was not built (reference source tree absent at build time)")
    ref = ReferenceKernels()
    if not ref.has_ce:
        pytest.skip("oracle/_ref was built without the loss-head kernels")
    torch.cuda.set_device(0)
    p = pkg()
    rows, cols, total = 96, 50257, 512
    z, tg = _case(oracle, rows, cols, 4711)
    tz_a, tz_b, tt = to_dev(z, z, tg)
    ga, gb = torch.empty_like(tz_a), torch.empty_like(tz_b)
    la, lb = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    p.chunked_logit_ce(tz_a, tt, la, total, grad_logits=ga)
    assert p.sync_status() == 0
    ref.chunked_logit_ce(tz_b, tt, gb, lb, total)
    assert _close(tz_a.cpu().numpy(), tz_b.cpu().numpy()) <= 1.0
    assert float((ga - gb).abs().max()) <= 3e-5 / total + 1e-9
    assert abs(float(la) - float(lb)) <= 1e-5 * abs(float(lb))
    probs_ref, grad_ref, loss_ref = oracle.chunked_ce(z, tg, total, train=True)   # and the oracle agrees with the reference
    assert _close(tz_b.cpu().numpy(), probs_ref) <= 1.0
    assert abs(float(lb) - loss_ref) <= 1e-5 * abs(loss_ref)
