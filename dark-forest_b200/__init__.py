"""dark-forest_b200: B200 (sm_100a) fused causal attention behind Dark Forest's launch API.

The product is the C-ABI library ``lib/libdarkforest_kernels.so`` (declared in
``include/darkforest_kernels.h``). This Python module is only the thin loader that the tests
and the benchmark use to reach that ABI: ctypes prototypes plus ``AttentionContext``, a mirror
of the reference's ``darkforest_cuda::AttentionContext`` (darkforest-cuda/src/lib.rs:1949-2368)
working on torch CUDA tensors. torch is used for device memory and streams, nothing else.

There is no CPU path: loading fails loudly when the CUDA library has not been built, and every
call needs CUDA tensors.

Because the directory name contains a hyphen, import it by path (see ``load_package`` in
``__graft_entry__.py``) under the module name ``dark_forest_b200``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libdarkforest_kernels.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "darkforest_kernels.h")

DF_OK = 0
DF_ERR_INVALID_ARG = 1
DF_ERR_UNSUPPORTED = 2
DF_ERR_CUDA = 3
DF_ERR_DEVICE_TIMEOUT = 4
DF_ERR_WORKSPACE = 5
DF_ERR_STATIC_SCRATCH = 6
DF_ERR_DEVICE_BOUNDS = 9
STATIC_SCRATCH_MAX_ROWS = 2097152
VARIANT_AUTO, VARIANT_SIMT, VARIANT_TENSOR = 0, 1, 2
OPT_FWD_PERSIST, OPT_FUSE_DELTA, OPT_BWD_OVERLAP, OPT_SCHED_TABLE, OPT_DISABLE_TENSOR, OPT_PDL, OPT_CE_VARIANT, OPT_LN_STAGED = range(8)

_P = ctypes.c_void_p
_U32 = ctypes.c_uint32
_F32 = ctypes.c_float
_I64 = ctypes.c_int64
_U64 = ctypes.c_uint64

# name -> (restype, argtypes); mirrors include/darkforest_kernels.h one to one
PROTOTYPES = {
    "launch_fused_attention": (None, [_P, _P, _P, _P, _U32, _U32, _F32, _U32]),
    "launch_fused_mha_forward": (None, [_P, _P, _P, _P, _U32, _U32, _U32, _F32, _U32]),
    "launch_attention_backward": (None, [_P] * 8 + [_U32, _U32, _F32, _U32]),
    "launch_fused_mha_backward": (None, [_P] * 8 + [_U32, _U32, _U32, _F32, _U32]),
    "darkforest_sync": (None, []),
    "launch_pos_embed_interpolate": (None, [_P, _P, _U32, _U32, _U32, _U32]),
    "launch_apply_rope": (None, [_P, _U32, _U32, _U32, _F32]),
    "launch_paged_copy_row": (None, [_P, _P, ctypes.c_int32, _U32, _U32, _U32]),
    "launch_paged_copy_row_f32_to_bf16": (None, [_P, _P, ctypes.c_int32, _U32, _U32, _U32]),
    "df_attn_apply_rope_rows": (ctypes.c_int, [_P, _U32, _U32, _U32, _U32, _F32, _P]),
    "df_attn_workspace_bytes": (ctypes.c_uint64, [ctypes.c_int, _U32, _U32, _U32, _U32, _U32]),
    "df_attn_schedule_build": (ctypes.c_int, [_P, ctypes.c_int, ctypes.c_int, _P, _P]),
    "df_attn_schedule_item": (ctypes.c_longlong, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_longlong]),
    "launch_fused_mha_decode_kv": (None, [_P, _P, _P, _P, _U32, _U32, _U32, _F32]),
    "launch_fused_mha_decode_kv_splitk": (None, [_P] * 7 + [_U32, _U32, _U32, _F32, _U32]),
    "launch_paged_mha_decode_kv": (None, [_P] * 5 + [_U32, _U32, _U32, _F32, _U32]),
    "launch_paged_mha_decode_kv_splitk": (None, [_P] * 8 + [_U32, _U32, _U32, _F32, _U32, _U32]),
    "launch_paged_mha_decode_kv_bf16": (None, [_P] * 5 + [_U32, _U32, _U32, _F32, _U32]),
    "df_attn_decode": (ctypes.c_int, [_P] * 8 + [_U32] * 4 + [_F32, _U32, _U32, _P]),
    "df_attn_forward": (ctypes.c_int, [_P] * 5 + [_U32] * 4 + [_F32, _U32, _P]),
    "df_attn_forward_block": (ctypes.c_int, [_P] * 5 + [_U32] * 5 + [_F32, _U32, _I64, _P]),
    "df_attn_forward_bf16": (ctypes.c_int, [_P] * 5 + [_U32] * 5 + [_F32, _U32, _I64, _U32, _P]),
    "df_attn_delta_bf16": (ctypes.c_int, [_P] * 3 + [_U32] * 4 + [_P]),
    "df_attn_backward_block_bf16": (ctypes.c_int, [_P] * 9 + [_U32] * 5 + [_F32, _U32, _I64, _U32, _P]),
    "df_attn_backward_bf16": (ctypes.c_int, [_P] * 10 + [_U32] * 4 + [_F32, _U32, _P]),
    "df_attn_delta": (ctypes.c_int, [_P] * 3 + [_U32] * 4 + [_P]),
    "df_attn_backward": (ctypes.c_int, [_P] * 10 + [_U32] * 4 + [_F32, _U32, _P]),
    "df_attn_backward_static_scratch": (ctypes.c_int, [_P] * 9 + [_U32] * 4 + [_F32, _U32, _P]),
    "df_attn_backward_block": (ctypes.c_int, [_P] * 9 + [_U32] * 5 + [_F32, _U32, _I64, _P]),
    "df_attn_merge_partials": (ctypes.c_int, [_P] * 4 + [_U32] * 4 + [_P]),
    "df_attn_accumulate": (ctypes.c_int, [_P, _P, _U64, _P]),
    "df_linear_qkv_forward": (ctypes.c_int, [_P] * 10 + [_U32] * 3 + [_P]),
    "df_linear_forward": (ctypes.c_int, [_P] * 5 + [_U32] * 3 + [_P]),
    "df_linear_gelu_forward": (ctypes.c_int, [_P] * 5 + [_U32] * 3 + [_P]),
    "launch_fused_chunked_logit_ce": (None, [_P] * 4 + [_U32] * 3),
    "launch_chunked_ce_eval": (None, [_P] * 3 + [_U32] * 3),
    "df_chunked_logit_ce": (ctypes.c_int, [_P] * 4 + [_U32] * 3 + [_P]),
    "launch_layernorm": (None, [_P] * 6 + [_U32, _U32]),
    "launch_layernorm_backward": (None, [_P] * 8 + [_U32, _U32]),
    "launch_gelu": (None, [_P, _P, _U32]),
    "launch_gelu_backward": (None, [_P, _P, _P, _U32]),
    "launch_adamw_update": (None, [_P] * 4 + [_U32] + [_F32] * 7),
    "df_layernorm_forward": (ctypes.c_int, [_P] * 6 + [_U32, _U32, _P]),
    "df_layernorm_backward": (ctypes.c_int, [_P] * 8 + [_U32, _U32, _P]),
    "df_gelu_forward": (ctypes.c_int, [_P, _P, _U64, _P]),
    "df_gelu_backward": (ctypes.c_int, [_P, _P, _P, _U64, _P]),
    "df_adamw_update": (ctypes.c_int, [_P] * 4 + [_U64] + [_F32] * 7 + [_P]),
    "df_adamw_plan": (_U64, [_P, _U32]),
    "df_adamw_update_multi": (ctypes.c_int, [_P, _U32, _U64] + [_F32] * 7 + [_P]),
    "df_attn_init": (ctypes.c_int, []),
    "df_attn_backward_profile": (ctypes.c_int, [_P] * 10 + [_U32] * 4 + [_F32, _U32, _P, _P, _P]),
    "df_attn_set_option": (ctypes.c_int, [ctypes.c_int, ctypes.c_int]),
    "df_attn_get_option": (ctypes.c_int, [ctypes.c_int]),
    "df_attn_set_variant": (ctypes.c_int, [ctypes.c_int]),
    "df_attn_forward_uses_tensor_cores": (ctypes.c_int, [_P] * 4 + [_U32] * 4),
    "df_attn_last_status": (ctypes.c_int, []),
    "df_attn_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "df_sync_status": (ctypes.c_int, []),
    "df_attn_selftest_wait_expiry": (ctypes.c_int, [_U32, _P]),
    "df_attn_selftest_bounds_check": (ctypes.c_int, [_P]),
    "df_attn_launch_count": (_U64, [ctypes.c_int]),
    "df_attn_build_info": (ctypes.c_char_p, []),
}

_lib = None


def build(verbose: bool = False) -> None:
    """Compile the CUDA library in-tree with nvcc for sm_100a (no GPU needed to compile)."""
    r = subprocess.run(["make", "-C", _HERE, "-j8"], capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode != 0:
        raise RuntimeError("building libdarkforest_kernels.so failed")


def lib() -> ctypes.CDLL:
    """The loaded C-ABI library. Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `make -C {_HERE}` "
                               "(the attention path has no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(L, name)  # AttributeError if the library does not export the symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class AttentionError(RuntimeError):
    pass


def _check(status: int) -> None:
    if status != DF_OK:
        raise AttentionError(f"attention call failed: {lib().df_attn_status_string(status).decode()} ({status})")


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise AttentionError("attention tensors must live on a CUDA device (no CPU path)")
    if not t.is_contiguous():
        raise AttentionError("attention tensors must be contiguous")
    return t.data_ptr()


def _stream_ptr(stream):
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return ctypes.c_void_p(s.cuda_stream)


def set_variant(v: int) -> int:
    return lib().df_attn_set_variant(v)


def set_option(option: int, value: int) -> int:
    """Process-wide tuning option (OPT_*); returns the previous value."""
    prev = lib().df_attn_set_option(option, value)
    if prev < 0 and option not in range(8):
        raise AttentionError(f"unknown option {option}")
    return prev


def init() -> None:
    """Creates the calling thread's side stream and events for the block backward on the current device."""
    _check(lib().df_attn_init())


def sync_status() -> int:
    return lib().df_sync_status()


def launch_count(reset: bool = False) -> int:
    return int(lib().df_attn_launch_count(1 if reset else 0))


# ------------------------------------------------------------------------------------------
# Batched, stream-aware calls on torch tensors: q,k,v,out [B,S,H*D] fp32, lse/delta [B,H,S] fp32
# ------------------------------------------------------------------------------------------
def forward(q, k, v, n_heads, scale, causal=True, out=None, lse=None, causal_shift=0, stream=None):
    import torch
    B, Sq, dm = q.shape
    Sk = k.shape[1]
    D = dm // n_heads
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((B, n_heads, Sq), dtype=torch.float32, device=q.device)
    _check(lib().df_attn_forward_block(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), B, n_heads, Sq, Sk, D,
                                       float(scale), int(bool(causal)), int(causal_shift), _stream_ptr(stream)))
    return out, lse


def decode(q, k, v, n_heads, cur_seq_len, scale, block_table=None, page_size=0, partials=None, max_chunks=0,
           out=None, stream=None):
    """One-token decode: q [H*D] fp32, k/v a contiguous cache [T_max, H*D] or, with block_table (int32
    tensor), a pool of pages of page_size rows; bf16 caches are recognised by dtype. partials =
    (m, l, o) scratch tensors for max_chunks states per head selects the split form."""
    import torch
    D = q.numel() // n_heads
    if out is None:
        out = torch.empty_like(q)
    pm, pl, po = partials if partials is not None else (None, None, None)
    _check(lib().df_attn_decode(_ptr(q), _ptr(k), _ptr(v), _ptr(block_table) if block_table is not None else None,
                                _ptr(out), _ptr(pm) if pm is not None else None, _ptr(pl) if pl is not None else None,
                                _ptr(po) if po is not None else None, int(max_chunks), n_heads, int(cur_seq_len), D,
                                float(scale), int(page_size), 1 if k.dtype == torch.bfloat16 else 0, _stream_ptr(stream)))
    return out


def forward_bf16(q, k, v, n_heads, scale, causal=True, out=None, lse=None, causal_shift=0, out_fp32=False, stream=None):
    """bf16 variant: q, k, v are torch.bfloat16 [B,S,H*D] (D = 64 or 128); out is bf16, or fp32 with
    out_fp32=True (ring partial results); lse is fp32."""
    import torch
    if q.dtype != torch.bfloat16:
        raise AttentionError("forward_bf16 needs bfloat16 tensors")
    B, Sq, dm = q.shape
    Sk = k.shape[1]
    if out is None:
        out = torch.empty(q.shape, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=q.device)
    if out.dtype != (torch.float32 if out_fp32 else torch.bfloat16):
        raise AttentionError("forward_bf16: out dtype does not match out_fp32")
    if lse is None:
        lse = torch.empty((B, n_heads, Sq), dtype=torch.float32, device=q.device)
    _check(lib().df_attn_forward_bf16(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), B, n_heads, Sq, Sk,
                                      dm // n_heads, float(scale), int(bool(causal)), int(causal_shift),
                                      int(bool(out_fp32)), _stream_ptr(stream)))
    return out, lse


def delta_bf16(out, d_out, n_heads, delta_buf=None, stream=None):
    import torch
    B, S, dm = out.shape
    if delta_buf is None:
        delta_buf = torch.empty((B, n_heads, S), dtype=torch.float32, device=out.device)
    _check(lib().df_attn_delta_bf16(_ptr(out), _ptr(d_out), _ptr(delta_buf), B, n_heads, S, dm // n_heads,
                                    _stream_ptr(stream)))
    return delta_buf


def backward_block_bf16(q, k, v, d_out, lse, delta_buf, n_heads, scale, causal=True, causal_shift=0, d_q=None, d_k=None,
                        d_v=None, out_fp32=False, stream=None):
    """Block form of the bf16 backward; gradients are bf16, or fp32 with out_fp32=True."""
    import torch
    B, Sq, dm = q.shape
    Sk = k.shape[1]
    gdt = torch.float32 if out_fp32 else torch.bfloat16
    d_q = torch.empty(q.shape, dtype=gdt, device=q.device) if d_q is None else d_q
    d_k = torch.empty(k.shape, dtype=gdt, device=q.device) if d_k is None else d_k
    d_v = torch.empty(v.shape, dtype=gdt, device=q.device) if d_v is None else d_v
    _check(lib().df_attn_backward_block_bf16(_ptr(q), _ptr(k), _ptr(v), _ptr(d_out), _ptr(lse), _ptr(delta_buf), _ptr(d_q),
                                             _ptr(d_k), _ptr(d_v), B, n_heads, Sq, Sk, dm // n_heads, float(scale),
                                             int(bool(causal)), int(causal_shift), int(bool(out_fp32)),
                                             _stream_ptr(stream)))
    return d_q, d_k, d_v


def backward_bf16(q, k, v, out, d_out, lse, n_heads, scale, causal=True, d_q=None, d_k=None, d_v=None, delta_buf=None,
                  stream=None):
    """bf16 variant of backward(): every [B,S,H*D] tensor is torch.bfloat16, lse and delta are fp32."""
    import torch
    B, S, dm = q.shape
    d_q = torch.empty_like(q) if d_q is None else d_q
    d_k = torch.empty_like(k) if d_k is None else d_k
    d_v = torch.empty_like(v) if d_v is None else d_v
    if delta_buf is None:
        delta_buf = torch.empty((B, n_heads, S), dtype=torch.float32, device=q.device)
    _check(lib().df_attn_backward_bf16(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(d_out), _ptr(lse), _ptr(d_q), _ptr(d_k),
                                       _ptr(d_v), _ptr(delta_buf), B, n_heads, S, dm // n_heads, float(scale),
                                       int(bool(causal)), _stream_ptr(stream)))
    return d_q, d_k, d_v


def delta(out, d_out, n_heads, delta_buf=None, stream=None):
    import torch
    B, S, dm = out.shape
    if delta_buf is None:
        delta_buf = torch.empty((B, n_heads, S), dtype=torch.float32, device=out.device)
    _check(lib().df_attn_delta(_ptr(out), _ptr(d_out), _ptr(delta_buf), B, n_heads, S, dm // n_heads,
                               _stream_ptr(stream)))
    return delta_buf


def backward(q, k, v, out, d_out, lse, n_heads, scale, causal=True, d_q=None, d_k=None, d_v=None,
             delta_buf=None, stream=None):
    import torch
    B, S, dm = q.shape
    d_q = torch.empty_like(q) if d_q is None else d_q
    d_k = torch.empty_like(k) if d_k is None else d_k
    d_v = torch.empty_like(v) if d_v is None else d_v
    if delta_buf is None:
        delta_buf = torch.empty((B, n_heads, S), dtype=torch.float32, device=q.device)
    _check(lib().df_attn_backward(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(d_out), _ptr(lse), _ptr(d_q),
                                  _ptr(d_k), _ptr(d_v), _ptr(delta_buf), B, n_heads, S, dm // n_heads,
                                  float(scale), int(bool(causal)), _stream_ptr(stream)))
    return d_q, d_k, d_v


def backward_profile(q, k, v, out, d_out, lse, n_heads, scale, causal=True, d_q=None, d_k=None, d_v=None,
                     delta_buf=None, stream=None):
    """backward() through df_attn_backward_profile: returns (d_q, d_k, d_v, ms_dq, ms_dkdv), the device time per
    launch of the dQ (+ delta) kernel and of the dK/dV kernel, each launched four times back to back between
    events (0, 0 when the SIMT path ran)."""
    import torch
    B, S, dm = q.shape
    d_q = torch.empty_like(q) if d_q is None else d_q
    d_k = torch.empty_like(k) if d_k is None else d_k
    d_v = torch.empty_like(v) if d_v is None else d_v
    if delta_buf is None:
        delta_buf = torch.empty((B, n_heads, S), dtype=torch.float32, device=q.device)
    ms_dq, ms_dkdv = ctypes.c_float(0.0), ctypes.c_float(0.0)
    _check(lib().df_attn_backward_profile(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(d_out), _ptr(lse), _ptr(d_q),
                                          _ptr(d_k), _ptr(d_v), _ptr(delta_buf), B, n_heads, S, dm // n_heads,
                                          float(scale), int(bool(causal)), _stream_ptr(stream),
                                          ctypes.cast(ctypes.byref(ms_dq), _P), ctypes.cast(ctypes.byref(ms_dkdv), _P)))
    return d_q, d_k, d_v, float(ms_dq.value), float(ms_dkdv.value)


def backward_static_scratch(q, k, v, out, d_out, lse, n_heads, scale, causal=True, d_q=None, d_k=None, d_v=None,
                            stream=None):
    """Backward through the entry point that takes no scratch argument and allocates nothing
    itself (the gradient tensors are allocated here, by the caller's side, only when not given).
    Raises AttentionError when batch*heads*seq_len exceeds STATIC_SCRATCH_MAX_ROWS."""
    import torch
    B, S, dm = q.shape
    d_q = torch.empty_like(q) if d_q is None else d_q
    d_k = torch.empty_like(k) if d_k is None else d_k
    d_v = torch.empty_like(v) if d_v is None else d_v
    _check(lib().df_attn_backward_static_scratch(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(d_out), _ptr(lse),
                                                 _ptr(d_q), _ptr(d_k), _ptr(d_v), B, n_heads, S, dm // n_heads,
                                                 float(scale), int(bool(causal)), _stream_ptr(stream)))
    return d_q, d_k, d_v


def backward_block(q, k, v, d_out, lse, delta_buf, n_heads, scale, causal=True, causal_shift=0, d_q=None,
                   d_k=None, d_v=None, stream=None):
    import torch
    B, Sq, dm = q.shape
    Sk = k.shape[1]
    d_q = torch.empty_like(q) if d_q is None else d_q
    d_k = torch.empty_like(k) if d_k is None else d_k
    d_v = torch.empty_like(v) if d_v is None else d_v
    _check(lib().df_attn_backward_block(_ptr(q), _ptr(k), _ptr(v), _ptr(d_out), _ptr(lse), _ptr(delta_buf),
                                        _ptr(d_q), _ptr(d_k), _ptr(d_v), B, n_heads, Sq, Sk, dm // n_heads,
                                        float(scale), int(bool(causal)), int(causal_shift),
                                        _stream_ptr(stream)))
    return d_q, d_k, d_v


def linear_qkv(x, wq, wk, wv, bq=None, bk=None, bv=None, q=None, k=None, v=None, stream=None):
    """q, k, v = x wq^T + bq, x wk^T + bk, x wv^T + bv in one launch. x [rows, in], w* [out, in], b* [out]."""
    import torch
    rows, fin = x.shape
    fout = wq.shape[0]
    q, k, v = (torch.empty((rows, fout), dtype=torch.float32, device=x.device) if t is None else t for t in (q, k, v))
    _check(lib().df_linear_qkv_forward(_ptr(x), _ptr(wq), _ptr(wk), _ptr(wv), _ptr(bq), _ptr(bk), _ptr(bv), _ptr(q), _ptr(k),
                                       _ptr(v), rows, fin, fout, _stream_ptr(stream)))
    return q, k, v


def linear(x, w, bias=None, residual=None, out=None, stream=None):
    """out = x w^T + bias + residual (bias, residual optional). x [rows, in], w [out, in]."""
    import torch
    rows, fin = x.shape
    fout = w.shape[0]
    if out is None:
        out = torch.empty((rows, fout), dtype=torch.float32, device=x.device)
    _check(lib().df_linear_forward(_ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), rows, fin, fout,
                                   _stream_ptr(stream)))
    return out


def linear_gelu(x, w, bias=None, pre_activation=None, out=None, keep_pre_activation=True, stream=None):
    """pre = x w^T + bias and out = gelu(pre) in one launch; returns (pre, out) (pre None with keep_pre_activation False)."""
    import torch
    rows, fin = x.shape
    fout = w.shape[0]
    if out is None:
        out = torch.empty((rows, fout), dtype=torch.float32, device=x.device)
    if pre_activation is None and keep_pre_activation:
        pre_activation = torch.empty((rows, fout), dtype=torch.float32, device=x.device)
    _check(lib().df_linear_gelu_forward(_ptr(x), _ptr(w), _ptr(bias), _ptr(pre_activation), _ptr(out), rows, fin, fout,
                                        _stream_ptr(stream)))
    return pre_activation, out


def chunked_logit_ce(logits, targets, loss, total_rows, grad_logits=None, stream=None):
    """Softmax + cross-entropy over a chunk: logits [rows, cols] fp32 (overwritten with probabilities when
    grad_logits is given), targets [rows] int32/uint32 token ids, loss [1] fp32 accumulator. grad_logits None: eval form."""
    rows, cols = logits.shape
    _check(lib().df_chunked_logit_ce(_ptr(logits), _ptr(targets), _ptr(grad_logits), _ptr(loss), rows, cols, int(total_rows),
                                     _stream_ptr(stream)))
    return loss


# ------------------------------------------------------------------------------------------
# LayerNorm, GELU and AdamW of the training step (the DeviceTensor methods of
# darkforest-cuda/src/lib.rs:769-790, 885-910, 993-1100, 1755-1800): torch tensors in, kernels of this library.
# ------------------------------------------------------------------------------------------
def layernorm(x, gamma=None, beta=None, out=None, means=None, rstds=None, stream=None):
    """LayerNorm over the last dimension of x [rows, cols] (fp32): returns (out, means, rstds), the statistics the
    backward needs (DeviceTensor::layernorm_into, lib.rs:1010-1040)."""
    import torch
    rows, cols = x.shape
    out = torch.empty_like(x) if out is None else out
    means = torch.empty(rows, dtype=torch.float32, device=x.device) if means is None else means
    rstds = torch.empty(rows, dtype=torch.float32, device=x.device) if rstds is None else rstds
    _check(lib().df_layernorm_forward(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(out), _ptr(means), _ptr(rstds), rows, cols,
                                      _stream_ptr(stream)))
    return out, means, rstds


def layernorm_backward(grad_out, x, gamma, means, rstds, grad_x=None, grad_gamma=None, grad_beta=None, stream=None):
    """Backward of layernorm (DeviceTensor::layernorm_backward_into, lib.rs:1074-1100): returns grad_x; the column sums
    are ADDED to grad_gamma / grad_beta when given (the caller zeroes them)."""
    import torch
    rows, cols = x.shape
    grad_x = torch.empty_like(x) if grad_x is None else grad_x
    _check(lib().df_layernorm_backward(_ptr(grad_out), _ptr(x), _ptr(gamma), _ptr(means), _ptr(rstds), _ptr(grad_x),
                                       _ptr(grad_gamma), _ptr(grad_beta), rows, cols, _stream_ptr(stream)))
    return grad_x


def gelu(x, out=None, stream=None):
    """tanh-form GELU (DeviceTensor::gelu_into, lib.rs:775-790)."""
    import torch
    out = torch.empty_like(x) if out is None else out
    _check(lib().df_gelu_forward(_ptr(x), _ptr(out), x.numel(), _stream_ptr(stream)))
    return out


def gelu_backward(grad_out, x, grad_x=None, stream=None):
    """grad_x = grad_out * gelu'(x) (DeviceTensor::gelu_backward_into, lib.rs:894-910)."""
    import torch
    grad_x = torch.empty_like(x) if grad_x is None else grad_x
    _check(lib().df_gelu_backward(_ptr(grad_out), _ptr(x), _ptr(grad_x), x.numel(), _stream_ptr(stream)))
    return grad_x


def adamw_update(parameter, first_moment, second_moment, gradient, lr, beta1, beta2, eps, weight_decay, bias_correction1,
                 bias_correction2, stream=None):
    """One AdamW step on one tensor, in place (DeviceTensor::adamw_update, lib.rs:1755-1800)."""
    _check(lib().df_adamw_update(_ptr(parameter), _ptr(first_moment), _ptr(second_moment), _ptr(gradient), parameter.numel(),
                                 float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), float(bias_correction1),
                                 float(bias_correction2), _stream_ptr(stream)))


class AdamwTensor(ctypes.Structure):
    """df_adamw_tensor_t of include/darkforest_kernels.h."""
    _fields_ = [("parameter", ctypes.c_void_p), ("first_moment", ctypes.c_void_p), ("second_moment", ctypes.c_void_p),
                ("gradient", ctypes.c_void_p), ("n", ctypes.c_uint64), ("first_chunk", ctypes.c_uint64)]


class AdamwPlan:
    """The tensor table of df_adamw_update_multi for a fixed list of (parameter, first_moment, second_moment, gradient)
    tensors: built and uploaded once, then every step is one launch over all of them."""

    def __init__(self, tensors):
        import torch
        self.tensors = list(tensors)  # keeps the tensors alive: the table holds raw pointers
        n = len(self.tensors)
        table = (AdamwTensor * n)()
        for e, (p, m, v, g) in zip(table, self.tensors):
            if not (p.numel() == m.numel() == v.numel() == g.numel()):
                raise AttentionError("parameter, moments and gradient differ in size")
            e.parameter, e.first_moment, e.second_moment, e.gradient, e.n = _ptr(p), _ptr(m), _ptr(v), _ptr(g), p.numel()
        self.n_tensors = n
        self.total_chunks = int(lib().df_adamw_plan(ctypes.cast(table, _P), n)) if n else 0
        host = torch.frombuffer(bytearray(bytes(table)), dtype=torch.uint8) if n else torch.empty(0, dtype=torch.uint8)
        self.table = host.to(self.tensors[0][0].device) if n else host

    def step(self, lr, beta1, beta2, eps, weight_decay, bias_correction1, bias_correction2, stream=None):
        _check(lib().df_adamw_update_multi(_ptr(self.table), self.n_tensors, self.total_chunks, float(lr), float(beta1),
                                           float(beta2), float(eps), float(weight_decay), float(bias_correction1),
                                           float(bias_correction2), _stream_ptr(stream)))


def merge_partials(o_a, lse_a, o_b, lse_b, n_heads, stream=None):
    B, S, dm = o_a.shape
    _check(lib().df_attn_merge_partials(_ptr(o_a), _ptr(lse_a), _ptr(o_b), _ptr(lse_b), B, n_heads, S,
                                        dm // n_heads, _stream_ptr(stream)))
    return o_a, lse_a


def accumulate(dst, src, stream=None):
    _check(lib().df_attn_accumulate(_ptr(dst), _ptr(src), dst.numel(), _stream_ptr(stream)))
    return dst


# ------------------------------------------------------------------------------------------
# Mirror of darkforest_cuda::AttentionContext (darkforest-cuda/src/lib.rs:1949-2368): same
# constructor checks, same method names and argument meaning, same legacy-stream semantics.
# ------------------------------------------------------------------------------------------
class AttentionContext:
    def __init__(self, n_heads: int, seq_len: int, d_head: int, probabilities=None):
        if d_head == 0 or d_head > 128:  # lib.rs:1981
            raise AttentionError("d_head must be in the range 1..=128")
        self.n_heads, self.seq_len, self.d_head = n_heads, seq_len, d_head
        self.d_model = n_heads * d_head
        self._prob = probabilities  # shared scratch holder: a one-element list, like the Arc<Mutex<Option<..>>>

    @classmethod
    def new_shared(cls, n_heads, seq_len, d_head, probabilities):
        return cls(n_heads, seq_len, d_head, probabilities)

    def _ensure_probabilities(self, device):
        """lib.rs:2019-2027: H*2*S*S floats, allocated on the first backward and then reused."""
        import torch
        holder = self._prob if self._prob is not None else [None]
        self._prob = holder
        if holder[0] is None:
            n = self.n_heads * 2 * self.seq_len * self.seq_len
            holder[0] = torch.empty(max(n, 1), dtype=torch.float32, device=device)
        return holder[0]

    def _check_shape(self, t, what):
        if tuple(t.shape) != (self.seq_len, self.d_model):  # lib.rs:2051, 2252-2257
            raise AttentionError(f"attention {what} shape mismatch")

    def forward_device_into(self, q, k, v, scale, causal, out):
        self._check_shape(out, "output")
        L = lib()
        import torch
        ptrs = [_ptr(t) for t in (q, k, v, out)]
        torch.cuda.current_stream().synchronize()  # the legacy symbols run on the legacy default stream
        if self.n_heads == 1:  # lib.rs:2055-2065
            L.launch_fused_attention(*ptrs, self.seq_len, self.d_head, float(scale), int(bool(causal)))
        else:
            L.launch_fused_mha_forward(*ptrs, self.n_heads, self.seq_len, self.d_head, float(scale),
                                       int(bool(causal)))
        _check(L.df_attn_last_status())

    def forward_device(self, q, k, v, scale, causal):
        import torch
        out = torch.zeros((self.seq_len, self.d_model), dtype=torch.float32, device=q.device)
        self.forward_device_into(q, k, v, scale, causal, out)
        return out

    def backward_device_into(self, q, k, v, d_out, scale, causal, d_q, d_k, d_v):
        for t, n in ((d_q, "d_q"), (d_k, "d_k"), (d_v, "d_v")):
            self._check_shape(t, n)
        L = lib()
        import torch
        ptrs = [_ptr(t) for t in (q, k, v, d_out, d_q, d_k, d_v)]
        ptrs.append(_ptr(self._ensure_probabilities(q.device)))
        torch.cuda.current_stream().synchronize()
        if self.n_heads == 1:  # lib.rs:2260-2274
            L.launch_attention_backward(*ptrs, self.seq_len, self.d_head, float(scale), int(bool(causal)))
        else:
            L.launch_fused_mha_backward(*ptrs, self.n_heads, self.seq_len, self.d_head, float(scale),
                                        int(bool(causal)))
        _check(L.df_attn_last_status())

    def backward_device(self, q, k, v, d_out, scale, causal):
        import torch
        d_q, d_k, d_v = (torch.zeros((self.seq_len, self.d_model), dtype=torch.float32, device=q.device)
                         for _ in range(3))
        self.backward_device_into(q, k, v, d_out, scale, causal, d_q, d_k, d_v)
        return d_q, d_k, d_v

    # host-slice variants (lib.rs:2295-2367): single head only, numpy in / numpy out, one
    # host->device copy of each input and one device->host copy of each result
    def forward(self, q, k, v, scale, causal, device="cuda"):
        import numpy as np
        import torch
        if self.n_heads != 1:
            raise AttentionError("host-slice forward is single-head only")
        tq, tk, tv = (torch.from_numpy(np.ascontiguousarray(x, np.float32).reshape(self.seq_len, self.d_model))
                      .to(device) for x in (q, k, v))
        out = self.forward_device(tq, tk, tv, scale, causal)
        _check(sync_status())
        return out.cpu().numpy().reshape(-1)

    def backward(self, q, k, v, d_out, scale, causal, device="cuda"):
        import numpy as np
        import torch
        if self.n_heads != 1:
            raise AttentionError("host-slice backward is single-head only")
        tq, tk, tv, tg = (torch.from_numpy(np.ascontiguousarray(x, np.float32).reshape(self.seq_len, self.d_model))
                          .to(device) for x in (q, k, v, d_out))
        grads = self.backward_device(tq, tk, tv, tg, scale, causal)
        _check(sync_status())
        return tuple(g.cpu().numpy().reshape(-1) for g in grads)


def fused_attention_forward(q, k, v, seq_len, d_head, scale, causal):
    """Free function of the reference (lib.rs:2371-2421): host slices in, host vector out."""
    return AttentionContext(1, seq_len, d_head).forward(q, k, v, scale, causal)


def attention_backward(q, k, v, d_out, seq_len, d_head, scale, causal):
    """Free function of the reference (lib.rs:2423-2479)."""
    return AttentionContext(1, seq_len, d_head).backward(q, k, v, d_out, scale, causal)
