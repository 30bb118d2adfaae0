// host_selftest.cpp — the reference's two GPU unit tests for this path, run through the C++ host
// layer: fused_attention_matches_cpu_reference (darkforest-cuda/src/lib.rs:2606-2628) and
// attention_backward_matches_cpu_and_finite_difference (lib.rs:2753-2829), with the same inputs
// and tolerances, plus a multi-head D=64 case that exercises the tensor-core kernels.
// The CPU expectations below are the test's own checker (as in the reference's test module).
// Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <vector>

#include "attention_context.hpp"

using std::vector;

static vector<float> cpu_forward(const vector<float> &q, const vector<float> &k, const vector<float> &v, size_t S, size_t H,
                                 size_t D, float scale, bool causal) {
  const size_t dm = H * D;
  vector<float> out(S * dm, 0.f);
  vector<double> w(S);
  for (size_t h = 0; h < H; ++h)
    for (size_t i = 0; i < S; ++i) {
      const size_t nk = causal ? i + 1 : S;
      double mx = -INFINITY, sum = 0;
      for (size_t j = 0; j < nk; ++j) {
        double dot = 0;
        for (size_t d = 0; d < D; ++d) dot += (double)q[i * dm + h * D + d] * k[j * dm + h * D + d];
        w[j] = dot * scale;
        mx = std::fmax(mx, w[j]);
      }
      for (size_t j = 0; j < nk; ++j) sum += (w[j] = std::exp(w[j] - mx));
      for (size_t j = 0; j < nk; ++j)
        for (size_t d = 0; d < D; ++d) out[i * dm + h * D + d] += (float)(w[j] / sum * v[j * dm + h * D + d]);
    }
  return out;
}

static int failures = 0;
static void expect(bool ok, const char *what) {
  std::printf("%s: %s\n", ok ? "ok  " : "FAIL", what);
  if (!ok) ++failures;
}

int main() {
  try {
    {  // forward known-answer test: S=5, D=4, single head
      const size_t S = 5, D = 4;
      vector<float> q(S * D), k(S * D), v(S * D);
      for (size_t i = 0; i < S * D; ++i) {
        q[i] = ((float)i - 7.0f) / 11.0f;
        k[i] = (3.0f - (float)i) / 13.0f;
        v[i] = std::sin((float)i);
      }
      const float scale = 1.0f / std::sqrt((float)D);
      const vector<float> got = df::fused_attention_forward(q, k, v, S, D, scale, true);
      const vector<float> want = cpu_forward(q, k, v, S, 1, D, scale, true);
      float err = 0;
      for (size_t i = 0; i < got.size(); ++i) err = std::fmax(err, std::fabs(got[i] - want[i]));
      expect(err <= 2e-4f, "fused_attention_matches_cpu_reference (|d| <= 2e-4)");
    }
    {  // backward: finite differences of sum(O * dO), delta 1e-3, tolerance 2e-3
      const size_t S = 4, D = 3;
      vector<float> q(S * D), k(S * D), v(S * D), g(S * D);
      for (size_t i = 0; i < S * D; ++i) {
        q[i] = ((float)i - 4.0f) / 9.0f;
        k[i] = (2.0f - (float)i) / 10.0f;
        v[i] = ((float)i + 1.0f) / 8.0f;
        g[i] = ((float)i - 3.0f) / 7.0f;
      }
      const float scale = 1.0f / std::sqrt((float)D);
      const df::AttentionContext::Gradients grads = df::attention_backward(q, k, v, g, S, D, scale, true);
      auto objective = [&](const vector<float> &q_, const vector<float> &k_, const vector<float> &v_) {
        const vector<float> o = df::fused_attention_forward(q_, k_, v_, S, D, scale, true);
        double s = 0;
        for (size_t i = 0; i < o.size(); ++i) s += (double)o[i] * g[i];
        return s;
      };
      const vector<float> *inputs[3] = {&q, &k, &v};
      const vector<float> *analytical[3] = {&grads.d_q, &grads.d_k, &grads.d_v};
      float worst = 0;
      for (int which = 0; which < 3; ++which)
        for (size_t idx = 0; idx < S * D; ++idx) {
          vector<float> plus[3] = {q, k, v}, minus[3] = {q, k, v};
          plus[which][idx] = (*inputs[which])[idx] + 1e-3f;
          minus[which][idx] = (*inputs[which])[idx] - 1e-3f;
          const double numerical = (objective(plus[0], plus[1], plus[2]) - objective(minus[0], minus[1], minus[2])) / 2e-3;
          worst = std::fmax(worst, (float)std::fabs((*analytical[which])[idx] - numerical));
        }
      expect(worst <= 2e-3f, "attention_backward_matches_finite_difference (|d| <= 2e-3)");
    }
    {  // multi-head, D = 64: device-tensor API, tensor-core kernels, both the legacy and the lse path
      const size_t H = 4, S = 300, D = 64, dm = H * D;
      vector<float> q(S * dm), k(S * dm), v(S * dm), g(S * dm);
      unsigned s = 12345u;
      auto rnd = [&]() { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
      for (size_t i = 0; i < S * dm; ++i) { q[i] = rnd() * 1.7f; k[i] = rnd() * 1.7f; v[i] = rnd() * 1.7f; g[i] = rnd(); }
      df::AttentionContext ctx(H, S, D);
      df::DeviceTensor dq_ = df::DeviceTensor::from_host(q, {S, dm}), dk_ = df::DeviceTensor::from_host(k, {S, dm}),
                       dv_ = df::DeviceTensor::from_host(v, {S, dm}), dg_ = df::DeviceTensor::from_host(g, {S, dm});
      df::DeviceTensor out = ctx.forward_device(dq_, dk_, dv_, 0.125f, true);
      df::cuda_sync();
      const vector<float> got = out.to_host(), want = cpu_forward(q, k, v, S, H, D, 0.125f, true);
      float err = 0;
      for (size_t i = 0; i < got.size(); ++i) err = std::fmax(err, std::fabs(got[i] - want[i]));
      expect(err <= 2e-3f, "multi-head D=64 forward through forward_device (|d| <= 2e-3, TF32)");
      // legacy backward (recomputes O, lse in the scratch) against the lse-saving path
      df::DeviceTensor a_q = df::DeviceTensor::zeros({S, dm}), a_k = df::DeviceTensor::zeros({S, dm}),
                       a_v = df::DeviceTensor::zeros({S, dm});
      ctx.backward_device_into(dq_, dk_, dv_, dg_, 0.125f, true, a_q, a_k, a_v);
      df::DeviceTensor o2 = df::DeviceTensor::zeros({S, dm}), lse = df::DeviceTensor::zeros({H, S}),
                       delta = df::DeviceTensor::zeros({H, S});
      df::DeviceTensor b_q = df::DeviceTensor::zeros({S, dm}), b_k = df::DeviceTensor::zeros({S, dm}),
                       b_v = df::DeviceTensor::zeros({S, dm});
      ctx.forward_lse_into(dq_, dk_, dv_, 0.125f, true, o2, lse);
      ctx.backward_from_lse_into(dq_, dk_, dv_, o2, dg_, lse, 0.125f, true, b_q, b_k, b_v, delta);
      df::cuda_sync();
      const vector<float> x = a_k.to_host(), y = b_k.to_host();
      float diff = 0, mag = 0;
      for (size_t i = 0; i < x.size(); ++i) { diff = std::fmax(diff, std::fabs(x[i] - y[i])); mag = std::fmax(mag, std::fabs(y[i])); }
      expect(mag > 0.01f && diff <= 1e-6f * std::fmax(1.0f, mag), "legacy backward == lse-saving backward (same kernels, same bits)");
    }
    {  // decode over a contiguous cache and over the same tokens in a shuffled paged pool (+ split-K)
      const size_t H = 6, D = 64, dm = H * D, T = 1000, T_max = 1024, page = 16, pages = T_max / page;
      vector<float> q(dm), k(T_max * dm), v(T_max * dm);
      unsigned s = 777u;
      auto rnd = [&]() { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
      for (auto &x : q) x = rnd() * 1.7f;
      for (size_t i = 0; i < T_max * dm; ++i) { k[i] = rnd() * 1.7f; v[i] = rnd() * 1.7f; }
      vector<float> want(dm);
      for (size_t h = 0; h < H; ++h) {  // plain two-pass softmax in double
        vector<double> sc(T);
        double mx = -1e300, sum = 0;
        for (size_t t = 0; t < T; ++t) {
          double d = 0;
          for (size_t e = 0; e < D; ++e) d += (double)q[h * D + e] * k[t * dm + h * D + e];
          sc[t] = d * 0.125;
          mx = std::fmax(mx, sc[t]);
        }
        for (size_t t = 0; t < T; ++t) { sc[t] = std::exp(sc[t] - mx); sum += sc[t]; }
        for (size_t e = 0; e < D; ++e) {
          double o = 0;
          for (size_t t = 0; t < T; ++t) o += sc[t] * v[t * dm + h * D + e];
          want[h * D + e] = (float)(o / sum);
        }
      }
      df::AttentionContext ctx(H, T_max, D);
      df::DeviceTensor dq_ = df::DeviceTensor::from_host(q, {dm}), dk_ = df::DeviceTensor::from_host(k, {T_max, dm}),
                       dv_ = df::DeviceTensor::from_host(v, {T_max, dm});
      df::DeviceTensor out = df::DeviceTensor::zeros({dm});
      ctx.decode_kv_into(dq_, dk_, dv_, T, 0.125f, out);
      df::cuda_sync();
      vector<float> got = out.to_host();
      float err = 0;
      for (size_t i = 0; i < dm; ++i) err = std::fmax(err, std::fabs(got[i] - want[i]));
      expect(err <= 2e-5f, "decode_kv_into over a contiguous cache (|d| <= 2e-5)");
      vector<int32_t> table(pages);
      for (size_t i = 0; i < pages; ++i) table[i] = (int32_t)((i * 37 + 11) % pages);  // 37 is coprime to 64
      vector<float> kp(T_max * dm), vp(T_max * dm);
      for (size_t lp = 0; lp < pages; ++lp)
        for (size_t i = 0; i < page * dm; ++i) {
          kp[(size_t)table[lp] * page * dm + i] = k[lp * page * dm + i];
          vp[(size_t)table[lp] * page * dm + i] = v[lp * page * dm + i];
        }
      df::DeviceTensor dkp = df::DeviceTensor::from_host(kp, {T_max, dm}), dvp = df::DeviceTensor::from_host(vp, {T_max, dm});
      int32_t *d_table = nullptr;
      df::check_cuda(cudaMalloc(&d_table, pages * sizeof(int32_t)), "cudaMalloc(block table)");
      df::check_cuda(cudaMemcpy(d_table, table.data(), pages * sizeof(int32_t), cudaMemcpyHostToDevice), "cudaMemcpy(block table)");
      df::DeviceTensor out2 = df::DeviceTensor::zeros({dm});
      ctx.decode_paged_kv_into(dq_, dkp, dvp, d_table, T, 0.125f, page, out2);
      df::cuda_sync();
      got = out2.to_host();
      err = 0;
      for (size_t i = 0; i < dm; ++i) err = std::fmax(err, std::fabs(got[i] - want[i]));
      expect(err <= 2e-5f, "decode_paged_kv_into through a shuffled block table (|d| <= 2e-5)");
      const size_t chunk = 128, chunks = (T + chunk - 1) / chunk;
      df::DeviceTensor pm = df::DeviceTensor::zeros({H * chunks}), pl = df::DeviceTensor::zeros({H * chunks}),
                       po = df::DeviceTensor::zeros({H * chunks * D}), out3 = df::DeviceTensor::zeros({dm});
      ctx.decode_paged_kv_splitk_into(dq_, dkp, dvp, d_table, pm, pl, po, T, 0.125f, page, chunk, out3);
      df::cuda_sync();
      got = out3.to_host();
      err = 0;
      for (size_t i = 0; i < dm; ++i) err = std::fmax(err, std::fabs(got[i] - want[i]));
      expect(err <= 2e-5f, "decode_paged_kv_splitk_into with caller partial buffers (|d| <= 2e-5)");
      cudaFree(d_table);
    }
    {  // device_tensor_gelu_matches_cpu (darkforest-cuda/src/lib.rs:2832-2848): five points, |d| <= 1e-5
      const vector<float> input = {-2.0f, -1.0f, 0.0f, 1.0f, 2.0f};
      df::DeviceTensor t = df::DeviceTensor::from_host(input, {5}), o = df::DeviceTensor::zeros({5});
      t.gelu_into(o);
      df::cuda_sync();
      const vector<float> got = o.to_host();
      float err = 0;
      for (size_t i = 0; i < 5; ++i) {
        const float v = input[i], c = std::sqrt(2.0f / 3.14159265358979f);
        err = std::fmax(err, std::fabs(got[i] - 0.5f * v * (1.0f + std::tanh(c * (v + 0.044715f * v * v * v)))));
      }
      expect(err <= 1e-5f, "device_tensor_gelu_matches_cpu (|d| <= 1e-5)");
    }
    {  // device_tensor_adamw_matches_cpu_reference (lib.rs:2679-2718) and two steps of lib.rs:2721-2751: |d| <= 1e-6
      const float lr = 1e-2f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f, wd = 0.1f;
      const vector<vector<float>> grads = {{0.2f, -0.4f, 0.8f}, {-0.1f, 0.3f, 0.2f}};
      vector<double> ep = {1.0, -2.0, 0.5}, em(3, 0.0), ev(3, 0.0);
      df::DeviceTensor p = df::DeviceTensor::from_host({1.0f, -2.0f, 0.5f}, {3}), m = df::DeviceTensor::zeros({3}),
                       v = df::DeviceTensor::zeros({3});
      float err = 0;
      for (int t = 1; t <= 2; ++t) {
        df::DeviceTensor g = df::DeviceTensor::from_host(grads[t - 1], {3});
        df::DeviceTensor::adamw_update(p, m, v, g, lr, b1, b2, eps, wd, 1.0f - std::pow(b1, (float)t), 1.0f - std::pow(b2, (float)t));
        df::cuda_sync();
        for (size_t i = 0; i < 3; ++i) {
          const double gi = grads[t - 1][i];
          em[i] = b1 * em[i] + (1.0 - b1) * gi;
          ev[i] = b2 * ev[i] + (1.0 - b2) * gi * gi;
          ep[i] = ep[i] * (1.0 - lr * wd) - lr * (em[i] / (1.0 - std::pow((double)b1, t))) / (std::sqrt(ev[i] / (1.0 - std::pow((double)b2, t))) + eps);
        }
        const vector<float> got = p.to_host();
        for (size_t i = 0; i < 3; ++i) err = std::fmax(err, (float)std::fabs(got[i] - ep[i]));
      }
      expect(err <= 1e-6f, "adamw_update matches two CPU steps (|d| <= 1e-6)");
      bool threw = false;
      try {
        df::DeviceTensor g4 = df::DeviceTensor::zeros({4});
        df::DeviceTensor::adamw_update(p, m, v, g4, lr, b1, b2, eps, wd, 0.1f, 0.001f);
      } catch (const df::Error &) { threw = true; }
      expect(threw, "adamw_update rejects mismatched shapes on the host");
    }
    {  // layernorm_into / layernorm_backward_into: a 37 x 768 matrix against a double-precision loop; the backward
       // zeroes grad_gamma / grad_beta first, like the reference's method (lib.rs:1088-1093)
      const size_t R = 37, C = 768;
      vector<float> x(R * C), go(R * C), gamma(C), beta(C);
      for (size_t i = 0; i < R * C; ++i) {
        x[i] = std::sin(0.37f * (float)i) * 1.7f + 0.3f;
        go[i] = std::cos(0.11f * (float)i);
      }
      for (size_t i = 0; i < C; ++i) {
        gamma[i] = 1.0f + 0.2f * std::sin((float)i);
        beta[i] = 0.1f * std::cos((float)i);
      }
      df::DeviceTensor dx = df::DeviceTensor::from_host(x, {R, C}), dgo = df::DeviceTensor::from_host(go, {R, C}),
                       dg = df::DeviceTensor::from_host(gamma, {C}), db = df::DeviceTensor::from_host(beta, {C}),
                       out = df::DeviceTensor::zeros({R, C}), means = df::DeviceTensor::zeros({R}), rstds = df::DeviceTensor::zeros({R}),
                       gx = df::DeviceTensor::zeros({R, C});
      df::DeviceTensor gg = df::DeviceTensor::from_host(vector<float>(C, 5.0f), {C}), gb = df::DeviceTensor::from_host(vector<float>(C, -3.0f), {C});
      dx.layernorm_into(&dg, &db, out, means, rstds);
      df::DeviceTensor::layernorm_backward_into(dgo, dx, &dg, means, rstds, gx, &gg, &gb);
      df::cuda_sync();
      const vector<float> o = out.to_host(), gxh = gx.to_host(), ggh = gg.to_host(), gbh = gb.to_host();
      vector<double> wg(C, 0.0), wb(C, 0.0);
      float e_out = 0, e_gx = 0, e_col = 0;
      for (size_t r = 0; r < R; ++r) {
        double mean = 0, var = 0, s1 = 0, s2 = 0;
        for (size_t c = 0; c < C; ++c) mean += x[r * C + c];
        mean /= C;
        for (size_t c = 0; c < C; ++c) var += (x[r * C + c] - mean) * (x[r * C + c] - mean);
        const double rstd = 1.0 / std::sqrt(var / C + 1e-5);
        for (size_t c = 0; c < C; ++c) {
          const double xh = (x[r * C + c] - mean) * rstd, ds = (double)go[r * C + c] * gamma[c];
          e_out = std::fmax(e_out, (float)std::fabs(o[r * C + c] - (xh * gamma[c] + beta[c])));
          s1 += ds;
          s2 += ds * xh;
          wg[c] += go[r * C + c] * xh;
          wb[c] += go[r * C + c];
        }
        for (size_t c = 0; c < C; ++c) {
          const double xh = (x[r * C + c] - mean) * rstd, ds = (double)go[r * C + c] * gamma[c];
          e_gx = std::fmax(e_gx, (float)std::fabs(gxh[r * C + c] - rstd / C * (C * ds - s1 - xh * s2)));
        }
      }
      for (size_t c = 0; c < C; ++c) {
        e_col = std::fmax(e_col, (float)std::fabs(ggh[c] - wg[c]));
        e_col = std::fmax(e_col, (float)std::fabs(gbh[c] - wb[c]));
      }
      expect(e_out <= 2e-5f * 4.0f, "layernorm_into (|d| <= 8e-5 on values up to 4)");
      expect(e_gx <= 2e-5f * 4.0f, "layernorm_backward_into grad_x (|d| <= 8e-5)");
      expect(e_col <= 2e-4f, "layernorm_backward_into zeroes, then fills grad_gamma / grad_beta (|d| <= 2e-4)");
      bool threw = false;
      try {
        df::DeviceTensor bad = df::DeviceTensor::zeros({R + 1});
        dx.layernorm_into(&dg, &db, out, bad, rstds);
      } catch (const df::Error &) { threw = true; }
      expect(threw, "layernorm_into rejects a statistics tensor of the wrong shape");
    }
    {  // constructor checks of the reference
      bool threw = false;
      try { df::AttentionContext bad(12, 128, 129); } catch (const df::Error &) { threw = true; }
      expect(threw, "d_head > 128 is rejected on the host");
    }
  } catch (const std::exception &e) {
    std::printf("FAIL: exception: %s\n", e.what());
    return 2;
  }
  return failures ? 1 : 0;
}
