/*
 * attn_oracle.c — CPU restatement of Dark Forest's attention arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are
 * compared against and the timed CPU baseline; nothing on the product path links
 * it, loads it or falls back to it.
 *
 * What it restates (paths are relative to the Dark Forest source tree):
 *   forward   darkforest-core/src/engine/static_gpt2.rs:2766-2798  (CPU engine,
 *             causal multi-head loop: scores for j<=i, max, exp/sum, inv_sum
 *             guard, weighted V sum) and the single-head test helper
 *             darkforest-cuda/src/lib.rs:2493-2527 (reference_attention).
 *   backward  darkforest-cuda/src/lib.rs:2529-2586 (reference_backward):
 *             P = softmax(scale*QK^T), dP = dO V^T, corr = sum(P*dP),
 *             dS = P*(dP-corr), dQ += scale*dS*K, dK += scale*dS*Q, dV += P*dO.
 *   layout    row-major [S, H*D], head h = columns h*D..(h+1)*D-1
 *             (darkforest-cuda/kernels/attention_fused.cu:60-66); a batch is B
 *             independent slabs [B][S][H*D].
 * Added on top of the reference formulas (the reference has no counterpart):
 *   lse_i   = max_i + ln(sum_j exp(s_ij - max_i))   (natural log)
 *   delta_i = sum_d dO_id * O_id
 *   the partial-result merge used by a sequence-parallel ring,
 *   which is the same max/exp rescale as the split-K decode reduction in
 *   darkforest-cuda/kernels/attention_fused.cu:714-760.
 *
 * Two arithmetic flavours: *_f32 keeps the reference's fp32 scalar arithmetic and
 * summation order; *_f64 accumulates in double and is used to budget rounding
 * error.  OpenMP parallelism is over (batch, head[, row]) units only, so the
 * per-row arithmetic order is unchanged by the thread count.
 *
 * Pinned against: the two closed-form known-answer tests of the reference
 * (darkforest-cuda/src/lib.rs:2606-2628 and :2753-2829, including its central
 * finite-difference check), torch's CPU scaled_dot_product_attention in fp64 (the
 * reference's own parity twin, scripts/verify_loss_parity.py:58), and, on a GPU,
 * the reference's CUDA kernels compiled from their own source into oracle/_ref.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define DF_EXPORT __attribute__((visibility("default")))

DF_EXPORT int df_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

DF_EXPORT void df_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* Seeded inputs: a counter-based generator so that any host (and the numpy    */
/* mirror in attn_oracle.py) produces the same N(0,1) stream for (seed, index). */
/* ------------------------------------------------------------------------- */
static inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

DF_EXPORT void df_oracle_fill_normal(float *dst, uint64_t n, uint64_t seed, uint64_t stream) {
  const uint64_t key = mix64(seed ^ (stream * 0xD1342543DE82EF95ull));
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    uint64_t r = mix64(key + (uint64_t)i * 0x2545F4914F6CDD1Dull);
    /* two 24-bit uniforms in (0,1] and [0,1) */
    double u1 = ((double)((r >> 40) & 0xFFFFFF) + 1.0) / 16777216.0;
    double u2 = (double)((r >> 8) & 0xFFFFFF) / 16777216.0;
    dst[i] = (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
  }
}

/* ------------------------------------------------------------------------- */
/* Forward, fp32-faithful.  One (b,h,row) at a time, exactly the loop order of  */
/* static_gpt2.rs:2768-2798.  lse may be NULL.                                  */
/* ------------------------------------------------------------------------- */
static void fwd_row_f32(const float *q, const float *k, const float *v, float *out, float *lse,
                        size_t S, size_t dm, size_t D, size_t i, float scale, int causal,
                        float *scores) {
  const size_t nk = causal ? i + 1 : S;
  float max_score = -INFINITY;
  for (size_t j = 0; j < nk; ++j) {
    float dot = 0.0f;
    for (size_t d = 0; d < D; ++d) dot += q[i * dm + d] * k[j * dm + d];
    scores[j] = dot * scale;
    if (scores[j] > max_score) max_score = scores[j];
  }
  float exp_sum = 0.0f;
  for (size_t j = 0; j < nk; ++j) {
    scores[j] = expf(scores[j] - max_score);
    exp_sum += scores[j];
  }
  const float inv_sum = exp_sum > 0.0f ? 1.0f / exp_sum : 0.0f;
  for (size_t d = 0; d < D; ++d) {
    float val = 0.0f;
    for (size_t j = 0; j < nk; ++j) val += (scores[j] * inv_sum) * v[j * dm + d];
    out[i * dm + d] = val;
  }
  if (lse) *lse = exp_sum > 0.0f ? max_score + logf(exp_sum) : -INFINITY;
}

/* q,k,v,out: [B][S][H*D]; lse: [B][H][S] (may be NULL). */
DF_EXPORT void df_oracle_mha_forward_f32(const float *q, const float *k, const float *v, float *out,
                                         float *lse, uint32_t B, uint32_t H, uint32_t S, uint32_t D,
                                         float scale, uint32_t causal) {
  const size_t dm = (size_t)H * D;
  const int64_t units = (int64_t)B * H * S;
#pragma omp parallel
  {
    float *scores = (float *)malloc(sizeof(float) * (S ? S : 1));
#pragma omp for schedule(dynamic, 16)
    for (int64_t u = 0; u < units; ++u) {
      /* heavy (late) causal rows first so dynamic scheduling balances */
      const size_t i = S - 1 - (size_t)(u % S);
      const size_t h = (size_t)(u / S) % H;
      const size_t b = (size_t)(u / S) / H;
      const size_t base = b * S * dm + h * D;
      fwd_row_f32(q + base, k + base, v + base, out + base,
                  lse ? lse + (b * H + h) * (size_t)S + i : NULL, S, dm, D, i, scale, (int)causal,
                  scores);
    }
    free(scores);
  }
}

/* Forward with double accumulation everywhere (error-budget reference). */
DF_EXPORT void df_oracle_mha_forward_f64(const float *q, const float *k, const float *v, float *out,
                                         float *lse, uint32_t B, uint32_t H, uint32_t S, uint32_t D,
                                         float scale, uint32_t causal) {
  const size_t dm = (size_t)H * D;
  const int64_t units = (int64_t)B * H * S;
#pragma omp parallel
  {
    double *scores = (double *)malloc(sizeof(double) * (S ? S : 1));
    double *acc = (double *)malloc(sizeof(double) * (D ? D : 1));
#pragma omp for schedule(dynamic, 16)
    for (int64_t u = 0; u < units; ++u) {
      const size_t i = S - 1 - (size_t)(u % S);
      const size_t h = (size_t)(u / S) % H;
      const size_t b = (size_t)(u / S) / H;
      const size_t base = b * S * dm + h * D;
      const float *qq = q + base, *kk = k + base, *vv = v + base;
      const size_t nk = causal ? i + 1 : S;
      double mx = -INFINITY;
      for (size_t j = 0; j < nk; ++j) {
        double dot = 0.0;
        for (size_t d = 0; d < D; ++d) dot += (double)qq[i * dm + d] * (double)kk[j * dm + d];
        scores[j] = dot * (double)scale;
        if (scores[j] > mx) mx = scores[j];
      }
      double sum = 0.0;
      for (size_t j = 0; j < nk; ++j) {
        scores[j] = exp(scores[j] - mx);
        sum += scores[j];
      }
      for (size_t d = 0; d < D; ++d) acc[d] = 0.0;
      for (size_t j = 0; j < nk; ++j)
        for (size_t d = 0; d < D; ++d) acc[d] += scores[j] * (double)vv[j * dm + d];
      const double inv = sum > 0.0 ? 1.0 / sum : 0.0;
      for (size_t d = 0; d < D; ++d) out[base + i * dm + d] = (float)(acc[d] * inv);
      if (lse) lse[(b * H + h) * (size_t)S + i] = sum > 0.0 ? (float)(mx + log(sum)) : -INFINITY;
    }
    free(scores);
    free(acc);
  }
}

/* ------------------------------------------------------------------------- */
/* Backward, fp32-faithful: lib.rs:2529-2586 applied per (batch, head).         */
/* dq, dk, dv are fully overwritten (the reference launcher memsets dK and dV   */
/* and overwrites dQ: attention_fused.cu:522-524, 510-515).                     */
/* ------------------------------------------------------------------------- */
DF_EXPORT void df_oracle_mha_backward_f32(const float *q, const float *k, const float *v,
                                          const float *d_out, float *d_q, float *d_k, float *d_v,
                                          uint32_t B, uint32_t H, uint32_t S, uint32_t D,
                                          float scale, uint32_t causal) {
  const size_t dm = (size_t)H * D;
  const int64_t units = (int64_t)B * H;
#pragma omp parallel
  {
    float *prob = (float *)malloc(sizeof(float) * (S ? S : 1));
    float *dprob = (float *)malloc(sizeof(float) * (S ? S : 1));
#pragma omp for schedule(dynamic, 1)
    for (int64_t u = 0; u < units; ++u) {
      const size_t h = (size_t)u % H, b = (size_t)u / H;
      const size_t base = b * S * dm + h * D;
      const float *qq = q + base, *kk = k + base, *vv = v + base, *go = d_out + base;
      float *gq = d_q + base, *gk = d_k + base, *gv = d_v + base;
      for (size_t r = 0; r < S; ++r)
        for (size_t d = 0; d < D; ++d) {
          gq[r * dm + d] = 0.0f;
          gk[r * dm + d] = 0.0f;
          gv[r * dm + d] = 0.0f;
        }
      for (size_t row = 0; row < S; ++row) {
        const size_t nk = causal ? row + 1 : S;
        float mx = -INFINITY;
        for (size_t key = 0; key < nk; ++key) {
          float dot = 0.0f;
          for (size_t d = 0; d < D; ++d) dot += qq[row * dm + d] * kk[key * dm + d];
          prob[key] = dot * scale;
          if (prob[key] > mx) mx = prob[key];
        }
        float norm = 0.0f;
        for (size_t key = 0; key < nk; ++key) norm += expf(prob[key] - mx);
        for (size_t key = 0; key < nk; ++key) prob[key] = expf(prob[key] - mx) / norm;
        for (size_t key = 0; key < nk; ++key) {
          float s = 0.0f;
          for (size_t d = 0; d < D; ++d) s += go[row * dm + d] * vv[key * dm + d];
          dprob[key] = s;
        }
        float corr = 0.0f;
        for (size_t key = 0; key < nk; ++key) corr += prob[key] * dprob[key];
        for (size_t key = 0; key < nk; ++key) {
          const float ds = prob[key] * (dprob[key] - corr);
          for (size_t d = 0; d < D; ++d) {
            gq[row * dm + d] += scale * ds * kk[key * dm + d];
            gk[key * dm + d] += scale * ds * qq[row * dm + d];
            gv[key * dm + d] += prob[key] * go[row * dm + d];
          }
        }
      }
    }
    free(prob);
    free(dprob);
  }
}

DF_EXPORT void df_oracle_mha_backward_f64(const float *q, const float *k, const float *v,
                                          const float *d_out, float *d_q, float *d_k, float *d_v,
                                          uint32_t B, uint32_t H, uint32_t S, uint32_t D,
                                          float scale, uint32_t causal) {
  const size_t dm = (size_t)H * D;
  const int64_t units = (int64_t)B * H;
#pragma omp parallel
  {
    double *prob = (double *)malloc(sizeof(double) * (S ? S : 1));
    double *dprob = (double *)malloc(sizeof(double) * (S ? S : 1));
    double *aq = (double *)malloc(sizeof(double) * ((size_t)S * D + 1));
    double *ak = (double *)malloc(sizeof(double) * ((size_t)S * D + 1));
    double *av = (double *)malloc(sizeof(double) * ((size_t)S * D + 1));
#pragma omp for schedule(dynamic, 1)
    for (int64_t u = 0; u < units; ++u) {
      const size_t h = (size_t)u % H, b = (size_t)u / H;
      const size_t base = b * S * dm + h * D;
      const float *qq = q + base, *kk = k + base, *vv = v + base, *go = d_out + base;
      memset(aq, 0, sizeof(double) * (size_t)S * D);
      memset(ak, 0, sizeof(double) * (size_t)S * D);
      memset(av, 0, sizeof(double) * (size_t)S * D);
      for (size_t row = 0; row < S; ++row) {
        const size_t nk = causal ? row + 1 : S;
        double mx = -INFINITY;
        for (size_t key = 0; key < nk; ++key) {
          double dot = 0.0;
          for (size_t d = 0; d < D; ++d) dot += (double)qq[row * dm + d] * (double)kk[key * dm + d];
          prob[key] = dot * (double)scale;
          if (prob[key] > mx) mx = prob[key];
        }
        double norm = 0.0;
        for (size_t key = 0; key < nk; ++key) {
          prob[key] = exp(prob[key] - mx);
          norm += prob[key];
        }
        double corr = 0.0;
        for (size_t key = 0; key < nk; ++key) {
          prob[key] /= norm;
          double s = 0.0;
          for (size_t d = 0; d < D; ++d) s += (double)go[row * dm + d] * (double)vv[key * dm + d];
          dprob[key] = s;
          corr += prob[key] * s;
        }
        for (size_t key = 0; key < nk; ++key) {
          const double ds = prob[key] * (dprob[key] - corr) * (double)scale;
          for (size_t d = 0; d < D; ++d) {
            aq[row * D + d] += ds * (double)kk[key * dm + d];
            ak[key * D + d] += ds * (double)qq[row * dm + d];
            av[key * D + d] += prob[key] * (double)go[row * dm + d];
          }
        }
      }
      for (size_t r = 0; r < S; ++r)
        for (size_t d = 0; d < D; ++d) {
          d_q[base + r * dm + d] = (float)aq[r * D + d];
          d_k[base + r * dm + d] = (float)ak[r * D + d];
          d_v[base + r * dm + d] = (float)av[r * D + d];
        }
    }
    free(prob);
    free(dprob);
    free(aq);
    free(ak);
    free(av);
  }
}

/* delta[b][h][i] = sum_d dO[b][i][h*D+d] * O[b][i][h*D+d] */
DF_EXPORT void df_oracle_delta_f32(const float *out, const float *d_out, float *delta, uint32_t B,
                                   uint32_t H, uint32_t S, uint32_t D) {
  const size_t dm = (size_t)H * D;
  const int64_t units = (int64_t)B * H * S;
#pragma omp parallel for schedule(static)
  for (int64_t u = 0; u < units; ++u) {
    const size_t i = (size_t)u % S, h = ((size_t)u / S) % H, b = ((size_t)u / S) / H;
    const size_t off = b * S * dm + i * dm + h * D;
    float s = 0.0f;
    for (size_t d = 0; d < D; ++d) s += d_out[off + d] * out[off + d];
    delta[(b * H + h) * (size_t)S + i] = s;
  }
}

/*
 * Merge two partial attention results over disjoint key sets (ring step):
 *   lse = logaddexp(lse_a, lse_b); O = e^(lse_a-lse) O_a + e^(lse_b-lse) O_b.
 * A partial with no visible key has lse = -inf and contributes nothing.
 * Result is written over (o_a, lse_a).
 */
DF_EXPORT void df_oracle_merge_partials_f32(float *o_a, float *lse_a, const float *o_b,
                                            const float *lse_b, uint32_t B, uint32_t H, uint32_t S,
                                            uint32_t D) {
  const size_t dm = (size_t)H * D;
  const int64_t units = (int64_t)B * H * S;
#pragma omp parallel for schedule(static)
  for (int64_t u = 0; u < units; ++u) {
    const size_t i = (size_t)u % S, h = ((size_t)u / S) % H, b = ((size_t)u / S) / H;
    const size_t off = b * S * dm + i * dm + h * D;
    const size_t li = (b * H + h) * (size_t)S + i;
    const float la = lse_a[li], lb = lse_b[li];
    const float mx = la > lb ? la : lb;
    if (mx == -INFINITY) {
      for (size_t d = 0; d < D; ++d) o_a[off + d] = 0.0f;
      continue;
    }
    const float wa = expf(la - mx), wb = expf(lb - mx);
    const float inv = 1.0f / (wa + wb);
    for (size_t d = 0; d < D; ++d) o_a[off + d] = (wa * o_a[off + d] + wb * o_b[off + d]) * inv;
    lse_a[li] = mx + logf(wa + wb);
  }
}

/* bf16 helpers (round-to-nearest-even), for the bf16 variant's inputs. */
DF_EXPORT void df_oracle_round_bf16(const float *src, float *dst, uint16_t *bits, uint64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    uint32_t u;
    memcpy(&u, &src[i], 4);
    uint32_t r = u + 0x7FFFu + ((u >> 16) & 1u);
    if ((u & 0x7F800000u) == 0x7F800000u) r = u; /* inf/nan pass through */
    r &= 0xFFFF0000u;
    if (bits) bits[i] = (uint16_t)(r >> 16);
    if (dst) memcpy(&dst[i], &r, 4);
  }
}

/* ------------------------------------------------------------------------------------------
 * Decode: one query token per head against a KV cache of `T` tokens.
 * Follows kernel_fused_mha_decode_kv (darkforest-cuda/kernels/attention_fused.cu:551-615) and
 * its paged form (:796-865): score_t = scale * q.k_t in fp32, online softmax in token order,
 * out = sum_t p_t v_t / l with the l > 0 guard. Token t lives at row t of a contiguous
 * [T_max, H*D] cache, or, when block_table != NULL, at row (t % page_size) of physical page
 * block_table[t / page_size] of a pool of pages of page_size rows.
 * accumulate64 != 0 sums in double (error budgeting). lse (may be NULL) receives the natural
 * logsumexp of the scaled scores per head.
 * ------------------------------------------------------------------------------------------ */
DF_EXPORT void df_oracle_decode(const float *q, const float *k, const float *v, float *out, float *lse,
                                const int32_t *block_table, uint32_t page_size, uint32_t H, uint32_t T,
                                uint32_t D, float scale, int accumulate64) {
  const size_t dm = (size_t)H * D;
#pragma omp parallel for schedule(static)
  for (int64_t hh = 0; hh < (int64_t)H; ++hh) {
    const size_t h = (size_t)hh;
    const float *qh = q + h * D;
    if (accumulate64) {
      double m = -INFINITY, l = 0.0, acc[128];
      for (size_t d = 0; d < D; ++d) acc[d] = 0.0;
      for (uint32_t t = 0; t < T; ++t) {
        const size_t row = block_table ? (size_t)block_table[t / page_size] * page_size + (t % page_size) : (size_t)t;
        const float *kt = k + row * dm + h * D, *vt = v + row * dm + h * D;
        double dot = 0.0;
        for (size_t d = 0; d < D; ++d) dot += (double)qh[d] * (double)kt[d];
        const double s = dot * (double)scale;
        const double m_new = s > m ? s : m;
        const double alpha = (m == -INFINITY) ? 0.0 : exp(m - m_new);
        const double p = exp(s - m_new);
        l = l * alpha + p;
        for (size_t d = 0; d < D; ++d) acc[d] = acc[d] * alpha + p * (double)vt[d];
        m = m_new;
      }
      for (size_t d = 0; d < D; ++d) out[h * D + d] = l > 0.0 ? (float)(acc[d] / l) : 0.0f;
      if (lse) lse[h] = l > 0.0 ? (float)(m + log(l)) : -INFINITY;
    } else {
      float m = -FLT_MAX, l = 0.0f, acc[128];
      for (size_t d = 0; d < D; ++d) acc[d] = 0.0f;
      for (uint32_t t = 0; t < T; ++t) {
        const size_t row = block_table ? (size_t)block_table[t / page_size] * page_size + (t % page_size) : (size_t)t;
        const float *kt = k + row * dm + h * D, *vt = v + row * dm + h * D;
        float dot = 0.0f;
        for (size_t d = 0; d < D; ++d) dot = fmaf(qh[d], kt[d], dot);
        const float s = dot * scale;
        const float m_new = s > m ? s : m;
        const float alpha = (m == -FLT_MAX) ? 0.0f : expf(m - m_new);
        const float p = expf(s - m_new);
        l = fmaf(l, alpha, p);
        for (size_t d = 0; d < D; ++d) acc[d] = fmaf(p, vt[d], acc[d] * alpha);
        m = m_new;
      }
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      for (size_t d = 0; d < D; ++d) out[h * D + d] = acc[d] * inv;
      if (lse) lse[h] = l > 0.0f ? m + logf(l) : -INFINITY;
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * Per-token helpers of the same reference file.
 * ------------------------------------------------------------------------------------------ */
/* kernel_pos_embed_interpolate (attention_fused.cu:1098-1125): row `pos` of the trained table, or the
 * linear interpolation at pos * (trained - 1) / (max - 1), in fp32 like the kernel. */
DF_EXPORT void df_oracle_pos_embed_interpolate(const float *table, float *out, uint32_t pos, uint32_t trained,
                                               uint32_t max_len, uint32_t d_model) {
  if (pos < trained && max_len <= trained) {
    for (uint32_t d = 0; d < d_model; ++d) out[d] = table[(size_t)pos * d_model + d];
    return;
  }
  const float stretch = (float)(trained - 1) / (float)(max_len - 1);
  const float at = (float)pos * stretch;
  const uint32_t lo = (uint32_t)at;
  const uint32_t hi = lo + 1 < trained ? lo + 1 : trained - 1;
  const float w = at - (float)lo;
  for (uint32_t d = 0; d < d_model; ++d)
    out[d] = (1.0f - w) * table[(size_t)lo * d_model + d] + w * table[(size_t)hi * d_model + d];
}

/* kernel_apply_rope (attention_fused.cu:1143-1166) on `rows` consecutive rows, row r at position
 * pos0 + r: pairs (2i, 2i+1) of every head rotate by (pos0 + r) * base^(-2i/d_head). single_pow != 0
 * evaluates the frequency with powf like the reference kernel, otherwise in double, rounded once. */
DF_EXPORT void df_oracle_apply_rope(float *qk, uint32_t pos0, uint32_t rows, uint32_t n_heads, uint32_t d_head,
                                    float base, int single_pow) {
  for (uint32_t r = 0; r < rows; ++r)
    for (uint32_t h = 0; h < n_heads; ++h)
      for (uint32_t i = 0; i < d_head / 2; ++i) {
        const float theta = single_pow ? powf(base, -2.0f * (float)i / (float)d_head)
                                       : (float)pow((double)base, -2.0 * (double)i / (double)d_head);
        const float angle = (float)(pos0 + r) * theta;
        const float c = cosf(angle), s = sinf(angle);
        float *p = qk + ((size_t)r * n_heads + h) * d_head + 2 * i;
        const float x0 = p[0], x1 = p[1];
        p[0] = x0 * c - x1 * s;
        p[1] = x0 * s + x1 * c;
      }
}

/*
 * Linear projection of the CPU engine, darkforest-core/src/engine/static_gpt2.rs:2717-2733 (cpu_linear):
 *   out[t, o] = (bias ? bias[o] : 0) + sum_i x[t, i] * w[o, i]      summed in index order, in fp32;
 * `residual` (may be NULL) is added afterwards, as the engine's add_into does after the output projection
 * (static_gpt2.rs:1339-1341). accumulate_f64 != 0: the sum runs in double (error budgeting).
 */
DF_EXPORT void df_oracle_linear(const float *x, const float *w, const float *bias, const float *residual, float *out,
                                uint32_t rows, uint32_t in_f, uint32_t out_f, int accumulate_f64) {
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < (int64_t)rows; ++t) {
    const float *xr = x + (size_t)t * in_f;
    for (uint32_t o = 0; o < out_f; ++o) {
      const float *wr = w + (size_t)o * in_f;
      float r;
      if (accumulate_f64) {
        double acc = bias ? (double)bias[o] : 0.0;
        for (uint32_t i = 0; i < in_f; ++i) acc += (double)xr[i] * (double)wr[i];
        r = (float)acc;
      } else {
        float acc = bias ? bias[o] : 0.0f;
        for (uint32_t i = 0; i < in_f; ++i) acc += xr[i] * wr[i];
        r = acc;
      }
      if (residual) r += residual[(size_t)t * out_f + o];
      out[(size_t)t * out_f + o] = r;
    }
  }
}

/*
 * Fused softmax + cross-entropy over a chunk of logits, restating the arithmetic of the reference's CUDA kernels
 * (the static step has no CPU form of its loss head): darkforest-cuda/kernels/softmax.cu:325-394
 * (kernel_fused_chunked_logit_ce) and :415-462 (kernel_chunked_ce_eval).
 *   row_max = max_i z_i;  e_i = exp(z_i - row_max);  p_i = e_i / sum_i e_i
 *   training: logits <- p, grad = (p - onehot(target)) / total_rows, loss += -log(max(p_target, 1e-12)) / total_rows
 *   eval (grad == NULL): loss += (-(z_target - row_max) + log(max(sum, 1e-12))) / total_rows, logits untouched
 * The fp32 flavour sums the exponentials the way the kernels do - 512 strided partial sums (thread t takes columns
 * t, t + 512, ..), then a pairwise tree - because a single running fp32 sum over a 50257-entry row drops every term
 * below half an ulp of the partial sum and ends up 1e-4 low; use_f64 != 0 sums in double. The loss is accumulated
 * row by row in double and added to *loss once (the GPU kernels add per row or per CTA with atomics, in no fixed order).
 */
static float df_sum_exp_like_the_kernel(const float *z, uint32_t cols, float mx) {
  float part[512];
  for (int t = 0; t < 512; ++t) part[t] = 0.0f;
  for (uint32_t i = 0; i < cols; ++i) part[i & 511u] += expf(z[i] - mx);
  for (int w = 256; w > 0; w >>= 1)
    for (int t = 0; t < w; ++t) part[t] += part[t + w];
  return part[0];
}
DF_EXPORT void df_oracle_chunked_ce(float *logits, const uint32_t *targets, float *grad, float *loss, uint32_t rows,
                                    uint32_t cols, uint32_t total_rows, int use_f64) {
  const float inv_rows = 1.0f / (float)total_rows;
  double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    float *z = logits + (size_t)r * cols;
    const uint32_t t = targets[r];
    float mx = -3.402823466e+38f;
    for (uint32_t i = 0; i < cols; ++i) mx = z[i] > mx ? z[i] : mx;
    if (use_f64) {
      double sum = 0.0;
      for (uint32_t i = 0; i < cols; ++i) sum += exp((double)z[i] - (double)mx);
      if (!grad) {
        if (t < cols) total += (-((double)z[t] - (double)mx) + log(sum > 1e-12 ? sum : 1e-12)) * (double)inv_rows;
        continue;
      }
      for (uint32_t i = 0; i < cols; ++i) {
        const double p = exp((double)z[i] - (double)mx) / sum;
        if (i == t) total += -log(p > 1e-12 ? p : 1e-12) * (double)inv_rows;
        z[i] = (float)p;
        grad[(size_t)r * cols + i] = (float)((p - (i == t ? 1.0 : 0.0)) * (double)inv_rows);
      }
    } else {
      const float sum = df_sum_exp_like_the_kernel(z, cols, mx);
      if (!grad) {
        if (t < cols) total += (double)((-(z[t] - mx) + logf(sum > 1e-12f ? sum : 1e-12f)) * inv_rows);
        continue;
      }
      const float inv_sum = 1.0f / sum;
      for (uint32_t i = 0; i < cols; ++i) {
        const float p = expf(z[i] - mx) * inv_sum;
        if (i == t) total += (double)(-logf(p > 1e-12f ? p : 1e-12f) * inv_rows);
        z[i] = p;
        grad[(size_t)r * cols + i] = (p - (i == t ? 1.0f : 0.0f)) * inv_rows;
      }
    }
  }
  *loss += (float)total;
}

/*
 * LayerNorm, GELU and AdamW of the training step, restating the arithmetic of the reference's CUDA kernels (the
 * static step has no CPU form of them): darkforest-cuda/kernels/layernorm.cu:25-95 (forward: mean, biased variance
 * of the centred values, rstd = 1 / sqrt(var + 1e-5), out = (x - mean) * rstd * gamma + beta), :113-184 (backward:
 * grad_x = rstd / n * (n * ds - sum(ds) - xhat * sum(ds * xhat)) with ds = grad_out * gamma; grad_gamma and
 * grad_beta ADD sum over rows of grad_out * xhat and of grad_out to what the buffers hold), kernels/elementwise.cu:
 * 180-228 (tanh form of GELU and its derivative) and kernels/matmul.cu:285-339 (AdamW with decoupled weight decay;
 * the two bias corrections are arguments). use_f64 != 0 runs every sum and every transcendental in double (error
 * budgeting); otherwise the arithmetic is fp32 with the sums taken in index order. gamma / beta / means / rstds /
 * grad_gamma / grad_beta may be NULL as in the kernels.
 */
DF_EXPORT void df_oracle_layernorm(const float *x, const float *gamma, const float *beta, float *out, float *means,
                                   float *rstds, uint32_t rows, uint32_t cols, int use_f64) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const float *xr = x + (size_t)r * cols;
    float *o = out + (size_t)r * cols;
    if (use_f64) {
      double s = 0.0, q = 0.0;
      for (uint32_t i = 0; i < cols; ++i) s += xr[i];
      const double mean = s / cols;
      for (uint32_t i = 0; i < cols; ++i) q += (xr[i] - mean) * (xr[i] - mean);
      const double rstd = 1.0 / sqrt(q / cols + 1e-5);
      if (means) means[r] = (float)mean;
      if (rstds) rstds[r] = (float)rstd;
      for (uint32_t i = 0; i < cols; ++i)
        o[i] = (float)((xr[i] - mean) * rstd * (gamma ? gamma[i] : 1.0) + (beta ? beta[i] : 0.0));
    } else {
      float s = 0.0f, q = 0.0f;
      for (uint32_t i = 0; i < cols; ++i) s += xr[i];
      const float mean = s / (float)cols;
      for (uint32_t i = 0; i < cols; ++i) {
        const float d = xr[i] - mean;
        q += d * d;
      }
      const float rstd = 1.0f / sqrtf(q / (float)cols + 1e-5f);
      if (means) means[r] = mean;
      if (rstds) rstds[r] = rstd;
      for (uint32_t i = 0; i < cols; ++i) o[i] = (xr[i] - mean) * rstd * (gamma ? gamma[i] : 1.0f) + (beta ? beta[i] : 0.0f);
    }
  }
}

DF_EXPORT void df_oracle_layernorm_backward(const float *grad_out, const float *x, const float *gamma, const float *means,
                                            const float *rstds, float *grad_x, float *grad_gamma, float *grad_beta,
                                            uint32_t rows, uint32_t cols, int use_f64) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < (int64_t)rows; ++r) {
    const float *xr = x + (size_t)r * cols, *dr = grad_out + (size_t)r * cols;
    float *gx = grad_x + (size_t)r * cols;
    if (use_f64) {
      const double mean = means[r], rstd = rstds[r], n = cols;
      double s1 = 0.0, s2 = 0.0;
      for (uint32_t i = 0; i < cols; ++i) {
        const double xh = (xr[i] - mean) * rstd, ds = (double)dr[i] * (gamma ? gamma[i] : 1.0);
        s1 += ds;
        s2 += ds * xh;
      }
      for (uint32_t i = 0; i < cols; ++i) {
        const double xh = (xr[i] - mean) * rstd, ds = (double)dr[i] * (gamma ? gamma[i] : 1.0);
        gx[i] = (float)(rstd / n * (n * ds - s1 - xh * s2));
      }
    } else {
      const float mean = means[r], rstd = rstds[r], n = (float)cols;
      float s1 = 0.0f, s2 = 0.0f;
      for (uint32_t i = 0; i < cols; ++i) {
        const float xh = (xr[i] - mean) * rstd, ds = dr[i] * (gamma ? gamma[i] : 1.0f);
        s1 += ds;
        s2 += ds * xh;
      }
      for (uint32_t i = 0; i < cols; ++i) {
        const float xh = (xr[i] - mean) * rstd, ds = dr[i] * (gamma ? gamma[i] : 1.0f);
        gx[i] = (rstd / n) * (n * ds - s1 - xh * s2);
      }
    }
  }
  /* column sums over the rows, in row order (the kernels add them with atomics, in no fixed order) */
  if (grad_gamma || grad_beta) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)cols; ++i) {
      if (use_f64) {
        double a = 0.0, b = 0.0;
        for (uint32_t r = 0; r < rows; ++r) {
          const double d = grad_out[(size_t)r * cols + i];
          a += d * (((double)x[(size_t)r * cols + i] - means[r]) * rstds[r]);
          b += d;
        }
        if (grad_gamma) grad_gamma[i] = (float)(grad_gamma[i] + a);
        if (grad_beta) grad_beta[i] = (float)(grad_beta[i] + b);
      } else {
        float a = 0.0f, b = 0.0f;
        for (uint32_t r = 0; r < rows; ++r) {
          const float d = grad_out[(size_t)r * cols + i];
          a += d * ((x[(size_t)r * cols + i] - means[r]) * rstds[r]);
          b += d;
        }
        if (grad_gamma) grad_gamma[i] += a;
        if (grad_beta) grad_beta[i] += b;
      }
    }
  }
}

DF_EXPORT void df_oracle_gelu(const float *x, float *out, uint64_t n, int use_f64) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    if (use_f64) {
      const double v = x[i], u = 0.7978845608028654 * (v + 0.044715 * v * v * v);
      out[i] = (float)(0.5 * v * (1.0 + tanh(u)));
    } else {
      const float v = x[i], u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      out[i] = 0.5f * v * (1.0f + tanhf(u));
    }
  }
}

DF_EXPORT void df_oracle_gelu_backward(const float *grad_out, const float *x, float *grad_x, uint64_t n, int use_f64) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    if (use_f64) {
      const double v = x[i], u = 0.7978845608028654 * (v + 0.044715 * v * v * v), t = tanh(u);
      const double du = 0.7978845608028654 * (1.0 + 3.0 * 0.044715 * v * v);
      grad_x[i] = (float)(grad_out[i] * (0.5 * (1.0 + t) + 0.5 * v * (1.0 - t * t) * du));
    } else {
      const float v = x[i], u = 0.7978845608028654f * (v + 0.044715f * v * v * v), t = tanhf(u);
      const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * v * v);
      grad_x[i] = grad_out[i] * (0.5f * (1.0f + t) + 0.5f * v * (1.0f - t * t) * du);
    }
  }
}

DF_EXPORT void df_oracle_adamw(float *p, float *m, float *v, const float *g, uint64_t n, float lr, float beta1, float beta2,
                               float eps, float weight_decay, float bc1, float bc2, int use_f64) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    if (use_f64) {
      const double mm = (double)beta1 * m[i] + (1.0 - (double)beta1) * g[i];
      const double vv = (double)beta2 * v[i] + (1.0 - (double)beta2) * ((double)g[i] * g[i]);
      m[i] = (float)mm;
      v[i] = (float)vv;
      p[i] = (float)(p[i] * (1.0 - (double)lr * weight_decay) - (double)lr * (mm / bc1) / (sqrt(vv / bc2) + eps));
    } else {
      const float mm = beta1 * m[i] + (1.0f - beta1) * g[i];
      const float vv = beta2 * v[i] + (1.0f - beta2) * (g[i] * g[i]);
      m[i] = mm;
      v[i] = vv;
      p[i] = p[i] * (1.0f - lr * weight_decay) - lr * (mm / bc1) / (sqrtf(vv / bc2) + eps);
    }
  }
}
