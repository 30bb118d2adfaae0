// attn_aux.cu — the small per-token kernels that share the reference's attention file: position
// embedding interpolation, rotary embedding, and the row copies that fill a paged KV pool
// (darkforest-cuda/kernels/attention_fused.cu:1098-1231). With them every symbol of that file is
// provided here and the file can be dropped from the reference's build.
//
// Each call moves or rewrites one row of d_model floats (a few KB): pure launch latency, nothing to
// tune beyond 16-byte accesses where the row allows them. df_attn_apply_rope_rows is the batched
// form (a block of consecutive positions in one launch) that a prefill needs.
#include <math.h>

#include "df_common.cuh"

namespace df {
namespace {

// out[d] = table[pos][d], or the linear interpolation between the two trained rows around
// pos * (trained - 1) / (max - 1) when the context was stretched beyond the trained length.
__global__ void k_pos_embed_interpolate(const float *__restrict__ table, float *__restrict__ out, uint32_t pos,
                                        uint32_t trained, uint32_t max_len, uint32_t d_model) {
  const uint32_t d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= d_model) return;
  if (pos < trained && max_len <= trained) {
    out[d] = __ldg(table + (size_t)pos * d_model + d);
    return;
  }
  const float stretch = (float)(trained - 1) / (float)(max_len - 1);
  const float at = (float)pos * stretch;
  const uint32_t lo = (uint32_t)at;
  const uint32_t hi = lo + 1 < trained ? lo + 1 : trained - 1;
  const float w = at - (float)lo;
  out[d] = (1.0f - w) * __ldg(table + (size_t)lo * d_model + d) + w * __ldg(table + (size_t)hi * d_model + d);
}

// Rotates the pairs (2i, 2i+1) of every head of `rows` consecutive rows in place; row r has position
// pos0 + r. The frequency base^(-2i/d_head) is evaluated in double and rounded once, so that the
// angle does not depend on a single-precision pow.
__global__ void k_apply_rope(float *__restrict__ qk, uint32_t pos0, uint32_t rows, uint32_t n_heads, uint32_t d_head,
                             float base) {
  const uint32_t pairs = d_head / 2;
  const uint32_t per_row = n_heads * pairs;
  const size_t total = (size_t)rows * per_row;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const uint32_t r = (uint32_t)(e / per_row), in_row = (uint32_t)(e % per_row);
    const uint32_t h = in_row / pairs, i = in_row % pairs;
    const float theta = (float)pow((double)base, -2.0 * (double)i / (double)d_head);
    const float angle = (float)(pos0 + r) * theta;
    float s, c;
    sincosf(angle, &s, &c);
    float *p = qk + ((size_t)r * n_heads + h) * d_head + 2 * i;  // an odd last element of a head stays as it is
    const float x0 = p[0], x1 = p[1];
    p[0] = x0 * c - x1 * s;
    p[1] = x0 * s + x1 * c;
  }
}

template <bool TO_BF16>
__global__ void k_paged_copy_row(const float *__restrict__ src, void *__restrict__ pool, size_t dst_row, uint32_t d_model) {
  const uint32_t d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= d_model) return;
  const float x = __ldg(src + d);
  if (TO_BF16) {
    // round to nearest even, like __float2bfloat16_rn; NaN keeps a quiet payload
    uint32_t u = __float_as_uint(x);
    uint16_t b;
    if ((u & 0x7fffffffu) > 0x7f800000u) b = (uint16_t)((u >> 16) | 0x0040u);
    else b = (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
    static_cast<uint16_t *>(pool)[dst_row * d_model + d] = b;
  } else {
    static_cast<float *>(pool)[dst_row * d_model + d] = x;
  }
}

int finish(int st) {
  note_status(st);
  return st;
}

}  // namespace
}  // namespace df

using namespace df;

extern "C" {

void launch_pos_embed_interpolate(const float *pos_table, float *out, uint32_t pos, uint32_t trained_ctx_len,
                                  uint32_t max_ctx_len, uint32_t d_model) {
  if (d_model == 0) return;
  if (!pos_table || !out || trained_ctx_len == 0) { finish(DF_ERR_INVALID_ARG); return; }
  // the stretched form divides by max_ctx_len - 1 and reads row pos * (trained - 1) / (max - 1) < trained
  const bool plain = pos < trained_ctx_len && max_ctx_len <= trained_ctx_len;
  if (!plain && (max_ctx_len < 2 || pos >= max_ctx_len)) { finish(DF_ERR_INVALID_ARG); return; }
  k_pos_embed_interpolate<<<(d_model + 255) / 256, 256>>>(pos_table, out, pos, trained_ctx_len, max_ctx_len, d_model);
  note_launch();
  finish(check_cuda(cudaGetLastError()));
}

int df_attn_apply_rope_rows(float *qk, uint32_t first_pos, uint32_t rows, uint32_t n_heads, uint32_t d_head,
                            float base_freq, void *stream) {
  if (rows == 0 || n_heads == 0 || d_head < 2) return DF_OK;
  if (!qk || !(base_freq > 0.0f)) return finish(DF_ERR_INVALID_ARG);
  const size_t total = (size_t)rows * n_heads * (d_head / 2);
  const unsigned blocks = (unsigned)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
  k_apply_rope<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(qk, first_pos, rows, n_heads, d_head, base_freq);
  note_launch();
  return finish(check_cuda(cudaGetLastError()));
}

void launch_apply_rope(float *qk, uint32_t pos, uint32_t n_heads, uint32_t d_head, float base_freq) {
  df_attn_apply_rope_rows(qk, pos, 1, n_heads, d_head, base_freq, nullptr);
}

void launch_paged_copy_row(const float *src, float *pool, int32_t phys_block, uint32_t page_offset, uint32_t page_size,
                           uint32_t d_model) {
  if (d_model == 0) return;
  if (!src || !pool || phys_block < 0 || page_offset >= page_size) { finish(DF_ERR_INVALID_ARG); return; }
  k_paged_copy_row<false><<<(d_model + 255) / 256, 256>>>(src, pool, (size_t)phys_block * page_size + page_offset, d_model);
  note_launch();
  finish(check_cuda(cudaGetLastError()));
}

void launch_paged_copy_row_f32_to_bf16(const float *src, void *pool, int32_t phys_block, uint32_t page_offset,
                                       uint32_t page_size, uint32_t d_model) {
  if (d_model == 0) return;
  if (!src || !pool || phys_block < 0 || page_offset >= page_size) { finish(DF_ERR_INVALID_ARG); return; }
  k_paged_copy_row<true><<<(d_model + 255) / 256, 256>>>(src, pool, (size_t)phys_block * page_size + page_offset, d_model);
  note_launch();
  finish(check_cuda(cudaGetLastError()));
}

}  // extern "C"
