//! Bindings for the B200 attention library, to sit beside (or replace parts of) `darkforest-cuda/src/kernels.rs`.
//!
//! Layout follows the reference shim: one `extern "C"` declaration per symbol of `include/darkforest_kernels.h`
//! (and, behind the `darkforest_ring` cfg, of `include/darkforest_ring.h`), and thin safe-signature wrappers in the
//! reference's style - `usize` -> `u32`, `bool` -> `u32`, `anyhow::Result` - for the entry points a `StaticGPT2`-like
//! caller needs. The four attention wrappers and the decode wrappers of the reference
//! (`kernels.rs:694-885`, `:1157-1350`) keep working unchanged against this library because the legacy symbols keep
//! their signatures; the wrappers below add what the reference has no symbol for: logsumexp-saving forward,
//! scratch-free backward, the fused projections and the ring.
//!
//! This file cannot be compiled where the library is built (no Rust toolchain there); `tests/test_abi.py` parses
//! the two `extern "C"` blocks and checks every name, argument count and argument type against the C headers.

#![allow(clippy::too_many_arguments)]

use anyhow::{anyhow, Result};
use std::os::raw::{c_char, c_void};

/// Status codes of the `df_*` entry points (`darkforest_kernels.h`).
pub const DF_OK: i32 = 0;
pub const DF_ERR_INVALID_ARG: i32 = 1;
pub const DF_ERR_UNSUPPORTED: i32 = 2;
pub const DF_ERR_CUDA: i32 = 3;
pub const DF_ERR_DEVICE_TIMEOUT: i32 = 4;
pub const DF_ERR_WORKSPACE: i32 = 5;
pub const DF_ERR_STATIC_SCRATCH: i32 = 6;
pub const DF_ERR_RING_TIMEOUT: i32 = 7;
pub const DF_ERR_NCCL: i32 = 8;
pub const DF_ERR_DEVICE_BOUNDS: i32 = 9;
pub const DF_STATIC_SCRATCH_MAX_ROWS: u64 = 2_097_152;

/// One entry of the tensor table of `df_adamw_update_multi` (`df_adamw_tensor_t`).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct DfAdamwTensor {
    pub parameter: *mut f32,
    pub first_moment: *mut f32,
    pub second_moment: *mut f32,
    pub gradient: *const f32,
    pub n: u64,
    pub first_chunk: u64,
}

#[cfg(darkforest_cuda_kernels)]
extern "C" {
    pub fn launch_fused_attention(
        q: *const f32, k: *const f32, v: *const f32, out: *mut f32, seq_len: u32, d_head: u32, scale: f32,
        causal: u32
    );
    pub fn launch_fused_mha_forward(
        q: *const f32, k: *const f32, v: *const f32, out: *mut f32, n_heads: u32, seq_len: u32, d_head: u32,
        scale: f32, causal: u32
    );
    pub fn launch_attention_backward(
        q: *const f32, k: *const f32, v: *const f32, d_out: *const f32, d_q: *mut f32, d_k: *mut f32,
        d_v: *mut f32, probabilities: *mut f32, seq_len: u32, d_head: u32, scale: f32, causal: u32
    );
    pub fn launch_fused_mha_backward(
        q: *const f32, k: *const f32, v: *const f32, d_out: *const f32, d_q: *mut f32, d_k: *mut f32,
        d_v: *mut f32, probabilities: *mut f32, n_heads: u32, seq_len: u32, d_head: u32, scale: f32, causal: u32
    );
    pub fn launch_fused_mha_decode_kv(
        q: *const f32, k_cache: *const f32, v_cache: *const f32, out: *mut f32, n_heads: u32, cur_seq_len: u32,
        d_head: u32, scale: f32
    );
    pub fn launch_fused_mha_decode_kv_splitk(
        q: *const f32, k_cache: *const f32, v_cache: *const f32, partial_m: *mut f32, partial_l: *mut f32,
        partial_o: *mut f32, out: *mut f32, n_heads: u32, cur_seq_len: u32, d_head: u32, scale: f32, chunk_size: u32
    );
    pub fn launch_paged_mha_decode_kv(
        q: *const f32, k_pool: *const f32, v_pool: *const f32, block_table: *const i32, out: *mut f32,
        n_heads: u32, cur_seq_len: u32, d_head: u32, scale: f32, page_size: u32
    );
    pub fn launch_paged_mha_decode_kv_splitk(
        q: *const f32, k_pool: *const f32, v_pool: *const f32, block_table: *const i32, partial_m: *mut f32,
        partial_l: *mut f32, partial_o: *mut f32, out: *mut f32, n_heads: u32, cur_seq_len: u32, d_head: u32,
        scale: f32, page_size: u32, chunk_size: u32
    );
    pub fn launch_paged_mha_decode_kv_bf16(
        q: *const f32, k_pool: *const c_void, v_pool: *const c_void, block_table: *const i32, out: *mut f32,
        n_heads: u32, cur_seq_len: u32, d_head: u32, scale: f32, page_size: u32
    );
    pub fn df_attn_decode(
        q: *const f32, k: *const c_void, v: *const c_void, block_table: *const i32, out: *mut f32,
        partial_m: *mut f32, partial_l: *mut f32, partial_o: *mut f32, max_chunks: u32, n_heads: u32,
        cur_seq_len: u32, d_head: u32, scale: f32, page_size: u32, kv_bf16: u32, stream: *mut c_void
    ) -> i32;
    pub fn launch_pos_embed_interpolate(
        pos_table: *const f32, out: *mut f32, pos: u32, trained_ctx_len: u32, max_ctx_len: u32, d_model: u32
    );
    pub fn launch_apply_rope(qk: *mut f32, pos: u32, n_heads: u32, d_head: u32, base_freq: f32);
    pub fn launch_paged_copy_row(
        src: *const f32, pool: *mut f32, phys_block: i32, page_offset: u32, page_size: u32, d_model: u32
    );
    pub fn launch_paged_copy_row_f32_to_bf16(
        src: *const f32, pool: *mut c_void, phys_block: i32, page_offset: u32, page_size: u32, d_model: u32
    );
    pub fn df_attn_apply_rope_rows(
        qk: *mut f32, first_pos: u32, rows: u32, n_heads: u32, d_head: u32, base_freq: f32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_schedule_build(weights: *const u32, n: i32, grid: i32, off: *mut u16, items: *mut u16) -> i32;
    pub fn df_attn_workspace_bytes(
        kind: i32, batch: u32, n_heads: u32, seq_len: u32, d_head: u32, chunk_size: u32
    ) -> u64;
    pub fn df_attn_schedule_item(round: i32, grid: i32, cta: i32, n_items: i64) -> i64;
    pub fn darkforest_sync();
    pub fn df_attn_forward(
        q: *const f32, k: *const f32, v: *const f32, out: *mut f32, lse: *mut f32, batch: u32, n_heads: u32,
        seq_len: u32, d_head: u32, scale: f32, causal: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_forward_block(
        q: *const f32, k: *const f32, v: *const f32, out: *mut f32, lse: *mut f32, batch: u32, n_heads: u32,
        seq_q: u32, seq_k: u32, d_head: u32, scale: f32, causal: u32, causal_shift: i64, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_forward_bf16(
        q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void, lse: *mut f32, batch: u32,
        n_heads: u32, seq_q: u32, seq_k: u32, d_head: u32, scale: f32, causal: u32, causal_shift: i64,
        out_fp32: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_backward_bf16(
        q: *const c_void, k: *const c_void, v: *const c_void, out: *const c_void, d_out: *const c_void,
        lse: *const f32, d_q: *mut c_void, d_k: *mut c_void, d_v: *mut c_void, delta: *mut f32, batch: u32,
        n_heads: u32, seq_len: u32, d_head: u32, scale: f32, causal: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_delta_bf16(
        out: *const c_void, d_out: *const c_void, delta: *mut f32, batch: u32, n_heads: u32, seq_len: u32,
        d_head: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_backward_block_bf16(
        q: *const c_void, k: *const c_void, v: *const c_void, d_out: *const c_void, lse: *const f32,
        delta: *const f32, d_q: *mut c_void, d_k: *mut c_void, d_v: *mut c_void, batch: u32, n_heads: u32,
        seq_q: u32, seq_k: u32, d_head: u32, scale: f32, causal: u32, causal_shift: i64, out_fp32: u32,
        stream: *mut c_void
    ) -> i32;
    pub fn df_attn_delta(
        out: *const f32, d_out: *const f32, delta: *mut f32, batch: u32, n_heads: u32, seq_len: u32, d_head: u32,
        stream: *mut c_void
    ) -> i32;
    pub fn df_attn_backward(
        q: *const f32, k: *const f32, v: *const f32, out: *const f32, d_out: *const f32, lse: *const f32,
        d_q: *mut f32, d_k: *mut f32, d_v: *mut f32, delta: *mut f32, batch: u32, n_heads: u32, seq_len: u32,
        d_head: u32, scale: f32, causal: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_init() -> i32;
    pub fn df_attn_backward_profile(
        q: *const f32, k: *const f32, v: *const f32, out: *const f32, d_out: *const f32, lse: *const f32,
        d_q: *mut f32, d_k: *mut f32, d_v: *mut f32, delta: *mut f32, batch: u32, n_heads: u32, seq_len: u32,
        d_head: u32, scale: f32, causal: u32, stream: *mut c_void, ms_dq: *mut f32, ms_dkdv: *mut f32
    ) -> i32;
    pub fn df_attn_backward_static_scratch(
        q: *const f32, k: *const f32, v: *const f32, out: *const f32, d_out: *const f32, lse: *const f32,
        d_q: *mut f32, d_k: *mut f32, d_v: *mut f32, batch: u32, n_heads: u32, seq_len: u32, d_head: u32,
        scale: f32, causal: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_backward_block(
        q: *const f32, k: *const f32, v: *const f32, d_out: *const f32, lse: *const f32, delta: *const f32,
        d_q: *mut f32, d_k: *mut f32, d_v: *mut f32, batch: u32, n_heads: u32, seq_q: u32, seq_k: u32, d_head: u32,
        scale: f32, causal: u32, causal_shift: i64, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_merge_partials(
        o_a: *mut f32, lse_a: *mut f32, o_b: *const f32, lse_b: *const f32, batch: u32, n_heads: u32, seq_len: u32,
        d_head: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_accumulate(dst: *mut f32, src: *const f32, n: u64, stream: *mut c_void) -> i32;
    pub fn df_linear_qkv_forward(
        x: *const f32, wq: *const f32, wk: *const f32, wv: *const f32, bq: *const f32, bk: *const f32,
        bv: *const f32, q: *mut f32, k: *mut f32, v: *mut f32, rows: u32, in_features: u32, out_features: u32,
        stream: *mut c_void
    ) -> i32;
    pub fn df_linear_forward(
        x: *const f32, w: *const f32, bias: *const f32, residual: *const f32, out: *mut f32, rows: u32,
        in_features: u32, out_features: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_linear_gelu_forward(
        x: *const f32, w: *const f32, bias: *const f32, pre_activation: *mut f32, out: *mut f32, rows: u32,
        in_features: u32, out_features: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_set_variant(variant: i32) -> i32;
    pub fn launch_fused_chunked_logit_ce(
        logits: *mut f32, targets: *const u32, grad_logits: *mut f32, loss: *mut f32, chunk_rows: u32, cols: u32,
        total_rows: u32
    );
    pub fn launch_chunked_ce_eval(logits: *mut f32, targets: *const u32, loss: *mut f32, chunk_rows: u32, cols: u32, total_rows: u32);
    pub fn df_chunked_logit_ce(
        logits: *mut f32, targets: *const u32, grad_logits: *mut f32, loss: *mut f32, chunk_rows: u32, cols: u32,
        total_rows: u32, stream: *mut c_void
    ) -> i32;
    pub fn launch_layernorm(
        x: *const f32, gamma: *const f32, beta: *const f32, out: *mut f32, means: *mut f32, rstds: *mut f32, batch: u32,
        features: u32
    );
    pub fn launch_layernorm_backward(
        grad_out: *const f32, x: *const f32, gamma: *const f32, means: *const f32, rstds: *const f32, grad_x: *mut f32,
        grad_gamma: *mut f32, grad_beta: *mut f32, batch: u32, features: u32
    );
    pub fn launch_gelu(x: *const f32, out: *mut f32, n: u32);
    pub fn launch_gelu_backward(grad_out: *const f32, x: *const f32, grad_x: *mut f32, n: u32);
    pub fn launch_adamw_update(
        parameter: *mut f32, first_moment: *mut f32, second_moment: *mut f32, gradient: *const f32, n: u32, lr: f32,
        beta1: f32, beta2: f32, eps: f32, weight_decay: f32, bias_correction1: f32, bias_correction2: f32
    );
    pub fn df_layernorm_forward(
        x: *const f32, gamma: *const f32, beta: *const f32, out: *mut f32, means: *mut f32, rstds: *mut f32, rows: u32,
        cols: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_layernorm_backward(
        grad_out: *const f32, x: *const f32, gamma: *const f32, means: *const f32, rstds: *const f32, grad_x: *mut f32,
        grad_gamma: *mut f32, grad_beta: *mut f32, rows: u32, cols: u32, stream: *mut c_void
    ) -> i32;
    pub fn df_gelu_forward(x: *const f32, out: *mut f32, n: u64, stream: *mut c_void) -> i32;
    pub fn df_gelu_backward(grad_out: *const f32, x: *const f32, grad_x: *mut f32, n: u64, stream: *mut c_void) -> i32;
    pub fn df_adamw_update(
        parameter: *mut f32, first_moment: *mut f32, second_moment: *mut f32, gradient: *const f32, n: u64, lr: f32,
        beta1: f32, beta2: f32, eps: f32, weight_decay: f32, bias_correction1: f32, bias_correction2: f32,
        stream: *mut c_void
    ) -> i32;
    pub fn df_adamw_plan(tensors_host: *mut DfAdamwTensor, n_tensors: u32) -> u64;
    pub fn df_adamw_update_multi(
        tensors_device: *const DfAdamwTensor, n_tensors: u32, total_chunks: u64, lr: f32, beta1: f32, beta2: f32, eps: f32,
        weight_decay: f32, bias_correction1: f32, bias_correction2: f32, stream: *mut c_void
    ) -> i32;
    pub fn df_attn_set_option(option: i32, value: i32) -> i32;
    pub fn df_attn_get_option(option: i32) -> i32;
    pub fn df_attn_forward_uses_tensor_cores(
        q: *const c_void, k: *const c_void, v: *const c_void, out: *const c_void, n_heads: u32, seq_q: u32,
        seq_k: u32, d_head: u32
    ) -> i32;
    pub fn df_attn_last_status() -> i32;
    pub fn df_attn_status_string(status: i32) -> *const c_char;
    pub fn df_attn_selftest_wait_expiry(budget_ms: u32, stream: *mut c_void) -> i32;
    pub fn df_attn_selftest_bounds_check(stream: *mut c_void) -> i32;
    pub fn df_sync_status() -> i32;
    pub fn df_attn_launch_count(reset: i32) -> u64;
    pub fn df_attn_build_info() -> *const c_char;
}

/// Opaque handle of `darkforest_ring.h`.
#[repr(C)]
pub struct DfRing {
    _private: [u8; 0],
}
pub const DF_RING_UNIQUE_ID_BYTES: usize = 128;
pub const DF_RING_LAYOUT_CONTIGUOUS: i32 = 0;
pub const DF_RING_LAYOUT_ZIGZAG: i32 = 1;
pub const DF_RING_LAYOUT_BALANCED: i32 = 2;

#[cfg(all(darkforest_cuda_kernels, darkforest_ring))]
extern "C" {
    pub fn df_ring_unique_id(id_out: *mut c_void) -> i32;
    pub fn df_ring_create(
        out: *mut *mut DfRing, unique_id: *const c_void, rank: i32, world: i32, layout: i32, n_heads: u32,
        local_len: u32, d_head: u32, bf16: i32, scale: f32, causal: i32, timeout_ms: u32
    ) -> i32;
    pub fn df_ring_workspace_bytes(ring: *const DfRing) -> u64;
    pub fn df_ring_forward(
        ring: *mut DfRing, q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void, lse: *mut f32,
        workspace: *mut c_void, workspace_bytes: u64, stream: *mut c_void
    ) -> i32;
    pub fn df_ring_backward(
        ring: *mut DfRing, q: *const c_void, k: *const c_void, v: *const c_void, out: *const c_void,
        d_out: *const c_void, lse: *const f32, d_q: *mut c_void, d_k: *mut c_void, d_v: *mut c_void,
        workspace: *mut c_void, workspace_bytes: u64, stream: *mut c_void
    ) -> i32;
    pub fn df_ring_wait(ring: *mut DfRing, stream: *mut c_void, timeout_ms: u32) -> i32;
    pub fn df_ring_last_nccl_result(ring: *const DfRing) -> i32;
    pub fn df_ring_destroy(ring: *mut DfRing) -> i32;
    pub fn df_ring_hop_blocks(rank: i32, world: i32, layout: i32, causal: i32, hop: i32, ops_out: *mut i32) -> i32;
}

#[cfg(darkforest_cuda_kernels)]
fn status(what: &str, st: i32) -> Result<()> {
    if st == DF_OK {
        return Ok(());
    }
    let msg = unsafe { std::ffi::CStr::from_ptr(df_attn_status_string(st)) };
    Err(anyhow!("{what}: {} ({st})", msg.to_string_lossy()))
}

/// Forward that also saves the logsumexp the backward needs: `out [B, S, H*D]`, `lse [B, H, S]`.
/// Extends `cuda_fused_mha_forward` (`kernels.rs:788-829`); launches on the legacy default stream like it.
pub fn cuda_attn_forward_lse(
    q: *const f32, k: *const f32, v: *const f32, out: *mut f32, lse: *mut f32,
    batch: usize, n_heads: usize, seq_len: usize, d_head: usize, scale: f32, causal: bool,
) -> Result<()> {
    #[cfg(darkforest_cuda_kernels)]
    unsafe {
        return status(
            "df_attn_forward",
            df_attn_forward(q, k, v, out, lse, batch as u32, n_heads as u32, seq_len as u32, d_head as u32, scale,
                causal as u32, std::ptr::null_mut()),
        );
    }
    #[cfg(not(darkforest_cuda_kernels))]
    Err(anyhow::Error::msg("CUDA kernels not compiled"))
}

/// Backward from the saved `out` and `lse`; `delta [B, H, S]` is scratch that the call fills. Two launches, no
/// `H*2*S*S` buffer. Extends `cuda_fused_mha_backward` (`kernels.rs:832-885`).
pub fn cuda_attn_backward_lse(
    q: *const f32, k: *const f32, v: *const f32, out: *const f32, d_out: *const f32, lse: *const f32,
    d_q: *mut f32, d_k: *mut f32, d_v: *mut f32, delta: *mut f32,
    batch: usize, n_heads: usize, seq_len: usize, d_head: usize, scale: f32, causal: bool,
) -> Result<()> {
    #[cfg(darkforest_cuda_kernels)]
    unsafe {
        return status(
            "df_attn_backward",
            df_attn_backward(q, k, v, out, d_out, lse, d_q, d_k, d_v, delta, batch as u32, n_heads as u32,
                seq_len as u32, d_head as u32, scale, causal as u32, std::ptr::null_mut()),
        );
    }
    #[cfg(not(darkforest_cuda_kernels))]
    Err(anyhow::Error::msg("CUDA kernels not compiled"))
}

/// The same for a host that has no `delta` slice to lend and may not allocate at step time: the row sums live in
/// an array inside the library (`batch * n_heads * seq_len <= DF_STATIC_SCRATCH_MAX_ROWS`, calls must not overlap).
pub fn cuda_attn_backward_static_scratch(
    q: *const f32, k: *const f32, v: *const f32, out: *const f32, d_out: *const f32, lse: *const f32,
    d_q: *mut f32, d_k: *mut f32, d_v: *mut f32,
    batch: usize, n_heads: usize, seq_len: usize, d_head: usize, scale: f32, causal: bool,
) -> Result<()> {
    #[cfg(darkforest_cuda_kernels)]
    unsafe {
        return status(
            "df_attn_backward_static_scratch",
            df_attn_backward_static_scratch(q, k, v, out, d_out, lse, d_q, d_k, d_v, batch as u32, n_heads as u32,
                seq_len as u32, d_head as u32, scale, causal as u32, std::ptr::null_mut()),
        );
    }
    #[cfg(not(darkforest_cuda_kernels))]
    Err(anyhow::Error::msg("CUDA kernels not compiled"))
}

/// Q, K, V projections of one layer in one launch: replaces the three `linear_into` calls of
/// `static_gpt2.rs:1324-1326` (three `cublasSgemm_v2` + three `cuda_add_bias`).
pub fn cuda_linear_qkv(
    x: *const f32, wq: *const f32, wk: *const f32, wv: *const f32, bq: *const f32, bk: *const f32, bv: *const f32,
    q: *mut f32, k: *mut f32, v: *mut f32, rows: usize, in_features: usize, out_features: usize,
) -> Result<()> {
    #[cfg(darkforest_cuda_kernels)]
    unsafe {
        return status(
            "df_linear_qkv_forward",
            df_linear_qkv_forward(x, wq, wk, wv, bq, bk, bv, q, k, v, rows as u32, in_features as u32,
                out_features as u32, std::ptr::null_mut()),
        );
    }
    #[cfg(not(darkforest_cuda_kernels))]
    Err(anyhow::Error::msg("CUDA kernels not compiled"))
}

/// `out = x w^T + bias + residual` in one launch: the output projection, its bias pass and the first residual add
/// (`static_gpt2.rs:1339-1341`). `bias` and `residual` may be null.
pub fn cuda_linear_bias_residual(
    x: *const f32, w: *const f32, bias: *const f32, residual: *const f32, out: *mut f32,
    rows: usize, in_features: usize, out_features: usize,
) -> Result<()> {
    #[cfg(darkforest_cuda_kernels)]
    unsafe {
        return status(
            "df_linear_forward",
            df_linear_forward(x, w, bias, residual, out, rows as u32, in_features as u32, out_features as u32,
                std::ptr::null_mut()),
        );
    }
    #[cfg(not(darkforest_cuda_kernels))]
    Err(anyhow::Error::msg("CUDA kernels not compiled"))
}

/// Step-boundary synchronisation that reports instead of aborting (`cuda_sync`, `kernels.rs:9-20`, aborts the
/// process through `darkforest_sync` on any CUDA error).
pub fn cuda_sync_checked() -> Result<()> {
    #[cfg(darkforest_cuda_kernels)]
    unsafe {
        return status("df_sync_status", df_sync_status());
    }
    #[cfg(not(darkforest_cuda_kernels))]
    Ok(())
}

/// One rank of the sequence-parallel ring (`darkforest_ring.h`). The unique id comes from rank 0
/// (`df_ring_unique_id`) over the host's own transport, e.g. `cluster::transport` (`transport.rs:16-22`).
#[cfg(all(darkforest_cuda_kernels, darkforest_ring))]
pub struct RingAttention {
    handle: *mut DfRing,
    workspace: *mut c_void,
    workspace_bytes: u64,
}

#[cfg(all(darkforest_cuda_kernels, darkforest_ring))]
impl RingAttention {
    /// `workspace` is caller-owned device memory of at least `workspace_bytes(..)` bytes, 256-byte aligned.
    pub fn new(
        unique_id: &[u8; DF_RING_UNIQUE_ID_BYTES], rank: usize, world: usize, layout: i32, n_heads: usize,
        local_len: usize, d_head: usize, bf16: bool, scale: f32, causal: bool, timeout_ms: u32,
    ) -> Result<Self> {
        let mut handle: *mut DfRing = std::ptr::null_mut();
        let st = unsafe {
            df_ring_create(&mut handle, unique_id.as_ptr() as *const c_void, rank as i32, world as i32, layout,
                n_heads as u32, local_len as u32, d_head as u32, bf16 as i32, scale, causal as i32, timeout_ms)
        };
        status("df_ring_create", st)?;
        Ok(Self { handle, workspace: std::ptr::null_mut(), workspace_bytes: 0 })
    }

    pub fn workspace_bytes(&self) -> u64 {
        unsafe { df_ring_workspace_bytes(self.handle) }
    }

    pub fn bind_workspace(&mut self, workspace: *mut c_void, bytes: u64) {
        self.workspace = workspace;
        self.workspace_bytes = bytes;
    }

    pub fn forward(&mut self, q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void, lse: *mut f32) -> Result<()> {
        let st = unsafe {
            df_ring_forward(self.handle, q, k, v, out, lse, self.workspace, self.workspace_bytes, std::ptr::null_mut())
        };
        status("df_ring_forward", st)
    }

    pub fn backward(
        &mut self, q: *const c_void, k: *const c_void, v: *const c_void, out: *const c_void, d_out: *const c_void,
        lse: *const f32, d_q: *mut c_void, d_k: *mut c_void, d_v: *mut c_void,
    ) -> Result<()> {
        let st = unsafe {
            df_ring_backward(self.handle, q, k, v, out, d_out, lse, d_q, d_k, d_v, self.workspace, self.workspace_bytes,
                std::ptr::null_mut())
        };
        status("df_ring_backward", st)
    }

    /// Bounded host-side wait; on a lost peer the communicator is aborted and an error comes back.
    pub fn wait(&mut self, timeout_ms: u32) -> Result<()> {
        status("df_ring_wait", unsafe { df_ring_wait(self.handle, std::ptr::null_mut(), timeout_ms) })
    }
}

#[cfg(all(darkforest_cuda_kernels, darkforest_ring))]
impl Drop for RingAttention {
    fn drop(&mut self) {
        unsafe {
            df_ring_destroy(self.handle);
        }
    }
}
