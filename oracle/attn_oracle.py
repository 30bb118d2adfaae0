"""CPU oracle for Dark Forest's attention path — TEST INFRASTRUCTURE ONLY.

Two things live here, both checkers and never part of the product path:

* ``numpy_*``: a direct numpy (float64) restatement of the formulas in
  darkforest-cuda/src/lib.rs:2493-2586 (``reference_attention`` / ``reference_backward``),
  used on small cases and to cross-check the C restatement.
* ``Oracle``: a ctypes loader for ``libdf_oracle.so`` (built from ``attn_oracle.c`` by the
  Makefile beside this file), the fp32-faithful restatement that parity tests compare the
  CUDA kernels against and that the benchmark times as its CPU baseline.

``ReferenceKernels`` loads the reference's own CUDA kernels
(darkforest-cuda/kernels/attention_fused.cu, compiled unmodified for sm_100a into
``oracle/_ref/`` by the same Makefile).  It needs a GPU and is used by GPU tests to pin
the restatement against the real implementation.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "libdf_oracle.so")
REFERENCE_SO = os.path.join(_HERE, "_ref", "libdf_reference_kernels.so")

_F = ctypes.POINTER(ctypes.c_float)
_U32 = ctypes.c_uint32


def build(force: bool = False) -> None:
    """Compile the C restatement (and oracle/_ref when the reference tree is present)."""
    if force or not os.path.exists(ORACLE_SO) or (
        os.path.getmtime(ORACLE_SO) < os.path.getmtime(os.path.join(_HERE, "attn_oracle.c"))
    ):
        subprocess.run(["make", "-C", _HERE, os.path.join(_HERE, "libdf_oracle.so")], check=True,
                       capture_output=True)
    if force or not os.path.exists(REFERENCE_SO):
        subprocess.run(["make", "-C", _HERE, "ref"], check=False, capture_output=True)


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_F)


# --------------------------------------------------------------------------------------
# Seeded inputs shared by every host: N(0,1) from a counter-based hash of (seed, stream, i)
# --------------------------------------------------------------------------------------
_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def numpy_fill_normal(n: int, seed: int, stream: int) -> np.ndarray:
    """numpy mirror of ``df_oracle_fill_normal`` (same values up to libm rounding)."""
    with np.errstate(over="ignore"):
        key = _mix64(np.array([seed], np.uint64) ^ (np.array([stream], np.uint64)
                                                    * np.uint64(0xD1342543DE82EF95)))
        r = _mix64(key + np.arange(n, dtype=np.uint64) * np.uint64(0x2545F4914F6CDD1D))
    u1 = (((r >> np.uint64(40)) & np.uint64(0xFFFFFF)).astype(np.float64) + 1.0) / 16777216.0
    u2 = ((r >> np.uint64(8)) & np.uint64(0xFFFFFF)).astype(np.float64) / 16777216.0
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


# --------------------------------------------------------------------------------------
# numpy restatement (float64), multi-head layout [B, S, H*D]
# --------------------------------------------------------------------------------------
def _heads(x: np.ndarray, H: int) -> np.ndarray:
    B, S, dm = x.shape
    return x.reshape(B, S, H, dm // H).transpose(0, 2, 1, 3).astype(np.float64)


def _unheads(x: np.ndarray) -> np.ndarray:
    B, H, S, D = x.shape
    return x.transpose(0, 2, 1, 3).reshape(B, S, H * D)


def numpy_forward(q, k, v, H, scale, causal=True):
    """Returns (out [B,S,H*D], lse [B,H,S]) in float64. lib.rs:2493-2527 per head."""
    qh, kh, vh = _heads(q, H), _heads(k, H), _heads(v, H)
    s = np.einsum("bhid,bhjd->bhij", qh, kh) * float(scale)
    S = s.shape[-1]
    if causal:
        s = np.where(np.tril(np.ones((S, S), bool)), s, -np.inf)
    m = s.max(-1, keepdims=True)
    w = np.exp(s - m)
    l = w.sum(-1, keepdims=True)
    o = np.einsum("bhij,bhjd->bhid", w / l, vh)
    return _unheads(o), (m + np.log(l))[..., 0]


def numpy_decode(q, k, v, H, T, scale):
    """float64 decode of one token over the first T rows of a contiguous cache; (out [H*D], lse [H])."""
    D = q.size // H
    qh = q.reshape(H, D).astype(np.float64)
    kh = k[:T].reshape(T, H, D).astype(np.float64)
    vh = v[:T].reshape(T, H, D).astype(np.float64)
    s = np.einsum("hd,thd->ht", qh, kh) * float(scale)
    m = s.max(-1, keepdims=True)
    w = np.exp(s - m)
    l = w.sum(-1, keepdims=True)
    o = np.einsum("ht,thd->hd", w / l, vh)
    return o.reshape(-1), (m + np.log(l))[:, 0]


def numpy_backward(q, k, v, d_out, H, scale, causal=True):
    """Returns (dq, dk, dv) in float64. lib.rs:2529-2586 per head."""
    qh, kh, vh, gh = _heads(q, H), _heads(k, H), _heads(v, H), _heads(d_out, H)
    s = np.einsum("bhid,bhjd->bhij", qh, kh) * float(scale)
    S = s.shape[-1]
    if causal:
        s = np.where(np.tril(np.ones((S, S), bool)), s, -np.inf)
    m = s.max(-1, keepdims=True)
    w = np.exp(s - m)
    p = w / w.sum(-1, keepdims=True)
    dp = np.einsum("bhid,bhjd->bhij", gh, vh)
    corr = (p * dp).sum(-1, keepdims=True)
    ds = p * (dp - corr)
    dq = np.einsum("bhij,bhjd->bhid", ds, kh) * float(scale)
    dk = np.einsum("bhij,bhid->bhjd", ds, qh) * float(scale)
    dv = np.einsum("bhij,bhid->bhjd", p, gh)
    return _unheads(dq), _unheads(dk), _unheads(dv)


# --------------------------------------------------------------------------------------
# C restatement
# --------------------------------------------------------------------------------------
class Oracle:
    """ctypes view of libdf_oracle.so. All arrays float32, layout [B, S, H*D]."""

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = L = ctypes.CDLL(path)
        fwd = [_F, _F, _F, _F, _F, _U32, _U32, _U32, _U32, ctypes.c_float, _U32]
        bwd = [_F] * 7 + [_U32, _U32, _U32, _U32, ctypes.c_float, _U32]
        for name in ("df_oracle_mha_forward_f32", "df_oracle_mha_forward_f64"):
            getattr(L, name).argtypes = fwd
            getattr(L, name).restype = None
        for name in ("df_oracle_mha_backward_f32", "df_oracle_mha_backward_f64"):
            getattr(L, name).argtypes = bwd
            getattr(L, name).restype = None
        L.df_oracle_delta_f32.argtypes = [_F, _F, _F, _U32, _U32, _U32, _U32]
        L.df_oracle_delta_f32.restype = None
        L.df_oracle_merge_partials_f32.argtypes = [_F, _F, _F, _F, _U32, _U32, _U32, _U32]
        L.df_oracle_merge_partials_f32.restype = None
        L.df_oracle_fill_normal.argtypes = [_F, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64]
        L.df_oracle_fill_normal.restype = None
        L.df_oracle_round_bf16.argtypes = [_F, _F, ctypes.POINTER(ctypes.c_uint16), ctypes.c_uint64]
        L.df_oracle_round_bf16.restype = None
        L.df_oracle_decode.argtypes = [_F, _F, _F, _F, _F, ctypes.POINTER(ctypes.c_int32), _U32, _U32, _U32, _U32,
                                       ctypes.c_float, ctypes.c_int]
        L.df_oracle_decode.restype = None
        L.df_oracle_pos_embed_interpolate.argtypes = [_F, _F, _U32, _U32, _U32, _U32]
        L.df_oracle_pos_embed_interpolate.restype = None
        L.df_oracle_apply_rope.argtypes = [_F, _U32, _U32, _U32, _U32, ctypes.c_float, ctypes.c_int]
        L.df_oracle_apply_rope.restype = None
        L.df_oracle_linear.argtypes = [_F, _F, _F, _F, _F, _U32, _U32, _U32, ctypes.c_int]
        L.df_oracle_linear.restype = None
        L.df_oracle_chunked_ce.argtypes = [_F, ctypes.POINTER(ctypes.c_uint32), _F, _F, _U32, _U32, _U32, ctypes.c_int]
        L.df_oracle_chunked_ce.restype = None
        _U64 = ctypes.c_uint64
        L.df_oracle_layernorm.argtypes = [_F] * 6 + [_U32, _U32, ctypes.c_int]
        L.df_oracle_layernorm.restype = None
        L.df_oracle_layernorm_backward.argtypes = [_F] * 8 + [_U32, _U32, ctypes.c_int]
        L.df_oracle_layernorm_backward.restype = None
        L.df_oracle_gelu.argtypes = [_F, _F, _U64, ctypes.c_int]
        L.df_oracle_gelu.restype = None
        L.df_oracle_gelu_backward.argtypes = [_F, _F, _F, _U64, ctypes.c_int]
        L.df_oracle_gelu_backward.restype = None
        L.df_oracle_adamw.argtypes = [_F, _F, _F, _F, _U64] + [ctypes.c_float] * 7 + [ctypes.c_int]
        L.df_oracle_adamw.restype = None
        L.df_oracle_max_threads.restype = ctypes.c_int
        L.df_oracle_set_threads.argtypes = [ctypes.c_int]

    @property
    def max_threads(self) -> int:
        return int(self.lib.df_oracle_max_threads())

    def set_threads(self, n: int) -> None:
        self.lib.df_oracle_set_threads(int(n))

    def fill_normal(self, shape, seed: int, stream: int) -> np.ndarray:
        a = np.empty(shape, np.float32)
        self.lib.df_oracle_fill_normal(_fp(a), a.size, seed, stream)
        return a

    @staticmethod
    def _dims(q: np.ndarray, H: int):
        B, S, dm = q.shape
        assert dm % H == 0
        return B, H, S, dm // H

    def forward(self, q, k, v, H, scale, causal=True, f64=False):
        B, H, S, D = self._dims(q, H)
        out = np.zeros_like(q)
        lse = np.zeros((B, H, S), np.float32)
        fn = self.lib.df_oracle_mha_forward_f64 if f64 else self.lib.df_oracle_mha_forward_f32
        fn(_fp(q), _fp(k), _fp(v), _fp(out), _fp(lse), B, H, S, D, scale, int(causal))
        return out, lse

    def backward(self, q, k, v, d_out, H, scale, causal=True, f64=False):
        B, H, S, D = self._dims(q, H)
        dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(q)
        fn = self.lib.df_oracle_mha_backward_f64 if f64 else self.lib.df_oracle_mha_backward_f32
        fn(_fp(q), _fp(k), _fp(v), _fp(d_out), _fp(dq), _fp(dk), _fp(dv), B, H, S, D, scale,
           int(causal))
        return dq, dk, dv

    def delta(self, out, d_out, H):
        B, H, S, D = self._dims(out, H)
        delta = np.zeros((B, H, S), np.float32)
        self.lib.df_oracle_delta_f32(_fp(out), _fp(d_out), _fp(delta), B, H, S, D)
        return delta

    def merge_partials(self, o_a, lse_a, o_b, lse_b, H):
        B, H, S, D = self._dims(o_a, H)
        o, l = o_a.copy(), lse_a.copy()
        self.lib.df_oracle_merge_partials_f32(_fp(o), _fp(l), _fp(o_b), _fp(lse_b), B, H, S, D)
        return o, l

    def decode(self, q, k, v, H, T, scale, block_table=None, page_size=0, f64=False):
        """One-token decode over the first T tokens of a KV cache. q [H*D]; k, v [rows, H*D]
        (a contiguous cache, or a pool of pages when block_table (int32) is given).
        Returns (out [H*D], lse [H]). attention_fused.cu:551-615, 796-865."""
        q = np.ascontiguousarray(q, np.float32).reshape(-1)
        D = q.size // H
        out = np.empty_like(q)
        lse = np.empty(H, np.float32)
        bt = None
        if block_table is not None:
            block_table = np.ascontiguousarray(block_table, np.int32)
            bt = block_table.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
        self.lib.df_oracle_decode(_fp(q), _fp(np.ascontiguousarray(k)), _fp(np.ascontiguousarray(v)), _fp(out), _fp(lse),
                                  bt, int(page_size), H, int(T), D, float(scale), 1 if f64 else 0)
        return out, lse

    def pos_embed_interpolate(self, table, pos, trained, max_len):
        """attention_fused.cu:1098-1125; table [trained, d_model] -> row [d_model]."""
        table = np.ascontiguousarray(table, np.float32)
        out = np.empty(table.shape[1], np.float32)
        self.lib.df_oracle_pos_embed_interpolate(_fp(table), _fp(out), int(pos), int(trained), int(max_len), table.shape[1])
        return out

    def apply_rope(self, qk, pos0, n_heads, d_head, base, single_pow=False):
        """attention_fused.cu:1143-1166 on rows [rows, n_heads*d_head] (a copy is rotated and returned)."""
        x = np.array(qk, np.float32, copy=True, order="C").reshape(-1, n_heads * d_head)
        self.lib.df_oracle_apply_rope(_fp(x), int(pos0), x.shape[0], n_heads, d_head, float(base), 1 if single_pow else 0)
        return x.reshape(np.shape(qk))

    def linear(self, x, w, bias=None, residual=None, f64=False):
        """out = x w^T + bias (+ residual): static_gpt2.rs:2717-2733. x [rows, in], w [out, in]."""
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        rows, fin = x.shape
        fout = w.shape[0]
        out = np.empty((rows, fout), np.float32)
        nul = ctypes.cast(None, _F)
        self.lib.df_oracle_linear(_fp(x), _fp(w), _fp(np.ascontiguousarray(bias, np.float32)) if bias is not None else nul,
                                  _fp(np.ascontiguousarray(residual, np.float32)) if residual is not None else nul,
                                  _fp(out), rows, fin, fout, 1 if f64 else 0)
        return out

    def chunked_ce(self, logits, targets, total_rows, train=True, f64=False):
        """softmax.cu:325-394 / 415-462 restated. Returns (probs, grad, loss) for the training form, (None, None, loss)
        for the eval form; loss is the chunk's contribution (a float)."""
        z = np.array(logits, np.float32, copy=True, order="C")
        t = np.ascontiguousarray(targets, np.uint32)
        rows, cols = z.shape
        loss = np.zeros(1, np.float32)
        grad = np.empty_like(z) if train else None
        self.lib.df_oracle_chunked_ce(_fp(z), t.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)),
                                      _fp(grad) if train else ctypes.cast(None, _F), _fp(loss), rows, cols, int(total_rows),
                                      1 if f64 else 0)
        return (z, grad, float(loss[0])) if train else (None, None, float(loss[0]))

    def layernorm(self, x, gamma=None, beta=None, f64=False):
        """layernorm.cu:25-95 restated. x [rows, cols] -> (out, means, rstds)."""
        x = np.ascontiguousarray(x, np.float32)
        rows, cols = x.shape
        out, means, rstds = np.empty_like(x), np.empty(rows, np.float32), np.empty(rows, np.float32)
        nul = ctypes.cast(None, _F)
        self.lib.df_oracle_layernorm(_fp(x), _fp(np.ascontiguousarray(gamma, np.float32)) if gamma is not None else nul,
                                     _fp(np.ascontiguousarray(beta, np.float32)) if beta is not None else nul, _fp(out),
                                     _fp(means), _fp(rstds), rows, cols, 1 if f64 else 0)
        return out, means, rstds

    def layernorm_backward(self, grad_out, x, gamma, means, rstds, grad_gamma0=None, grad_beta0=None, f64=False):
        """layernorm.cu:113-184 restated: returns (grad_x, grad_gamma, grad_beta); the column sums are added to
        grad_gamma0 / grad_beta0 (zeros when not given), as the kernel adds to what its buffers hold."""
        x = np.ascontiguousarray(x, np.float32)
        d = np.ascontiguousarray(grad_out, np.float32)
        rows, cols = x.shape
        gx = np.empty_like(x)
        gg = np.zeros(cols, np.float32) if grad_gamma0 is None else np.array(grad_gamma0, np.float32, copy=True)
        gb = np.zeros(cols, np.float32) if grad_beta0 is None else np.array(grad_beta0, np.float32, copy=True)
        nul = ctypes.cast(None, _F)
        self.lib.df_oracle_layernorm_backward(_fp(d), _fp(x), _fp(np.ascontiguousarray(gamma, np.float32)) if gamma is not None else nul,
                                              _fp(np.ascontiguousarray(means, np.float32)), _fp(np.ascontiguousarray(rstds, np.float32)),
                                              _fp(gx), _fp(gg), _fp(gb), rows, cols, 1 if f64 else 0)
        return gx, gg, gb

    def gelu(self, x, f64=False):
        """elementwise.cu:180-193 restated (tanh form)."""
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        self.lib.df_oracle_gelu(_fp(x), _fp(out), x.size, 1 if f64 else 0)
        return out

    def gelu_backward(self, grad_out, x, f64=False):
        """elementwise.cu:201-215 restated."""
        x = np.ascontiguousarray(x, np.float32)
        d = np.ascontiguousarray(grad_out, np.float32)
        gx = np.empty_like(x)
        self.lib.df_oracle_gelu_backward(_fp(d), _fp(x), _fp(gx), x.size, 1 if f64 else 0)
        return gx

    def adamw(self, p, m, v, g, lr, beta1, beta2, eps, weight_decay, bc1, bc2, f64=False):
        """matmul.cu:285-339 restated: returns updated copies (p, m, v)."""
        p, m, v = (np.array(a, np.float32, copy=True, order="C") for a in (p, m, v))
        g = np.ascontiguousarray(g, np.float32)
        self.lib.df_oracle_adamw(_fp(p), _fp(m), _fp(v), _fp(g), p.size, lr, beta1, beta2, eps, weight_decay, bc1, bc2,
                                 1 if f64 else 0)
        return p, m, v

    def round_bf16(self, x: np.ndarray):
        """Returns (x rounded to bf16 as float32, raw uint16 bits)."""
        dst = np.empty_like(x)
        bits = np.empty(x.shape, np.uint16)
        self.lib.df_oracle_round_bf16(_fp(np.ascontiguousarray(x)), _fp(dst),
                                      bits.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), x.size)
        return dst, bits


# --------------------------------------------------------------------------------------
# The reference's own CUDA kernels (GPU only)
# --------------------------------------------------------------------------------------
class ReferenceKernels:
    """Launches the unmodified reference kernels on torch CUDA tensors (legacy stream).

    Signatures: darkforest-cuda/kernels/attention_fused.cu:223-226, 233-237, 361-366, 518-521.
    The multi-head kernels are only correct for d_head <= 64 (two register slots per lane).
    """

    def __init__(self, path: str = REFERENCE_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = L = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        P = ctypes.c_void_p
        L.launch_fused_attention.argtypes = [P, P, P, P, _U32, _U32, ctypes.c_float, _U32]
        L.launch_fused_mha_forward.argtypes = [P, P, P, P, _U32, _U32, _U32, ctypes.c_float, _U32]
        L.launch_attention_backward.argtypes = [P] * 8 + [_U32, _U32, ctypes.c_float, _U32]
        L.launch_fused_mha_backward.argtypes = [P] * 8 + [_U32, _U32, _U32, ctypes.c_float, _U32]
        for n in ("launch_fused_attention", "launch_fused_mha_forward",
                  "launch_attention_backward", "launch_fused_mha_backward"):
            getattr(L, n).restype = None
        L.launch_fused_mha_decode_kv.argtypes = [P, P, P, P, _U32, _U32, _U32, ctypes.c_float]
        L.launch_fused_mha_decode_kv.restype = None
        self.has_ce = hasattr(L, "launch_fused_chunked_logit_ce")
        if self.has_ce:
            L.launch_fused_chunked_logit_ce.argtypes = [P, P, P, P, _U32, _U32, _U32]
            L.launch_fused_chunked_logit_ce.restype = None
            L.launch_chunked_ce_eval.argtypes = [P, P, P, _U32, _U32, _U32]
            L.launch_chunked_ce_eval.restype = None

        self.has_step = hasattr(L, "launch_layernorm")
        if self.has_step:
            L.launch_layernorm.argtypes = [P] * 6 + [_U32, _U32]
            L.launch_layernorm_backward.argtypes = [P] * 8 + [_U32, _U32]
            L.launch_gelu.argtypes = [P, P, _U32]
            L.launch_gelu_backward.argtypes = [P, P, P, _U32]
            L.launch_adamw_update.argtypes = [P] * 4 + [_U32] + [ctypes.c_float] * 7
            for n in ("launch_layernorm", "launch_layernorm_backward", "launch_gelu", "launch_gelu_backward", "launch_adamw_update"):
                getattr(L, n).restype = None

    def chunked_logit_ce(self, logits, targets, grad, loss, total_rows):
        """softmax.cu:396-410 (training form, grad given) or :469-480 (eval form, grad None), on torch tensors."""
        import torch
        rows, cols = logits.shape
        torch.cuda.synchronize()
        if grad is not None:
            self.lib.launch_fused_chunked_logit_ce(logits.data_ptr(), targets.data_ptr(), grad.data_ptr(), loss.data_ptr(),
                                                   rows, cols, total_rows)
        else:
            self.lib.launch_chunked_ce_eval(logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), rows, cols, total_rows)
        torch.cuda.synchronize()

    def decode_kv(self, q, k_cache, v_cache, H, T, scale):
        """attention_fused.cu:617-626 (one warp per head)."""
        import torch
        out = torch.empty_like(q)
        torch.cuda.synchronize()
        self.lib.launch_fused_mha_decode_kv(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                            H, T, q.numel() // H, scale)
        torch.cuda.synchronize()
        return out

    def mha_forward(self, q, k, v, H, scale, causal=True):
        import torch
        S, dm = q.shape
        out = torch.empty_like(q)
        torch.cuda.synchronize()
        self.lib.launch_fused_mha_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                          H, S, dm // H, scale, int(causal))
        torch.cuda.synchronize()
        return out

    def mha_backward(self, q, k, v, d_out, H, scale, causal=True):
        import torch
        S, dm = q.shape
        dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        scratch = torch.empty(H * 2 * S * S, dtype=torch.float32, device=q.device)
        torch.cuda.synchronize()
        self.lib.launch_fused_mha_backward(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                           d_out.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                           dv.data_ptr(), scratch.data_ptr(), H, S, dm // H, scale,
                                           int(causal))
        torch.cuda.synchronize()
        return dq, dk, dv
