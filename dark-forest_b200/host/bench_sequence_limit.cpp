// bench_sequence_limit.cpp — C++ twin of darkforest-core/src/bin/bench_sequence_limit.rs:
// the attention forward in isolation, H = 12, D = 64, fp32, causal, swept over
// S = 8K ... 2M with the reference's protocol (bench_sequence_limit.rs:52-74, 135-208, 222-227):
// four [S, 768] tensors, a warm-up launch only for S <= 16384, 3 timed launches for S <= 16384
// and 1 above, CUDA events, median, FLOPs = 2*H*S^2*D, JSON with the reference's schema.
// Differences, all stated in the output: the launch limit is a flag (--max-timed, default 131072 as
// in the reference; the B200 can go further), inputs can be seeded N(0,1) instead of the
// reference's all-zero tensors (--random), and the result path is a flag.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "attention_context.hpp"

struct Result {
  size_t seq_len;
  double latency_ms;  // < 0: not measured
  double vram_allocated_mb, free_vram_mb, tflops;
  std::string status;
};

static void fill_normal(df::DeviceTensor &t, unsigned long long seed) {
  // host-side seeded N(0,1) (Box-Muller over a 64-bit mix), uploaded once; not in any timed region
  std::vector<float> h(t.numel());
  unsigned long long s = seed;
  auto next = [&]() { s += 0x9E3779B97F4A7C15ull; unsigned long long z = s; z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
                      z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31); };
  for (size_t i = 0; i < h.size(); ++i) {
    const unsigned long long r = next();
    const double u1 = ((double)((r >> 40) & 0xFFFFFF) + 1.0) / 16777216.0, u2 = (double)((r >> 8) & 0xFFFFFF) / 16777216.0;
    h[i] = (float)(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
  }
  df::check_cuda(cudaMemcpy(t.as_mut_ptr(), h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice), "upload");
}

int main(int argc, char **argv) {
  size_t max_timed = 131072;
  bool random_inputs = false;
  std::string out_path = "kernel_scaling_results.json";
  size_t max_seq = 2097152;
  for (int i = 1; i < argc; ++i) {
    if (!std::strcmp(argv[i], "--max-timed") && i + 1 < argc) max_timed = std::strtoull(argv[++i], nullptr, 10);
    else if (!std::strcmp(argv[i], "--max-seq") && i + 1 < argc) max_seq = std::strtoull(argv[++i], nullptr, 10);
    else if (!std::strcmp(argv[i], "--random")) random_inputs = true;
    else if (!std::strcmp(argv[i], "--out") && i + 1 < argc) out_path = argv[++i];
    else { std::fprintf(stderr, "usage: %s [--max-timed S] [--max-seq S] [--random] [--out file.json]\n", argv[0]); return 2; }
  }
  try {
    const auto mem0 = df::get_memory_info();
    const double free_mb = mem0.first / 1048576.0, total_mb = mem0.second / 1048576.0;
    cudaDeviceProp prop;
    df::check_cuda(cudaGetDeviceProperties(&prop, 0), "cudaGetDeviceProperties");
    std::printf("Sequence Length Limit benchmark on %s: %.2f MB free / %.2f MB total\n", prop.name, free_mb, total_mb);
    const size_t n_heads = 12, d_head = 64, d_model = n_heads * d_head;
    const float scale = 1.0f / std::sqrt((float)d_head);
    const bool causal = true;
    std::vector<Result> results;
    for (size_t s = 8192; s <= max_seq; s *= 2) {
      std::printf("Testing Sequence Length S = %9zu ... ", s);
      std::fflush(stdout);
      const double theoretical_mb = 4.0 * s * d_model * sizeof(float) / 1048576.0;
      const size_t free_before = df::get_memory_info().first;
      df::DeviceTensor q, k, v, out;
      try {
        q = df::DeviceTensor::zeros({s, d_model});
        k = df::DeviceTensor::zeros({s, d_model});
        v = df::DeviceTensor::zeros({s, d_model});
        out = df::DeviceTensor::zeros({s, d_model});
      } catch (const df::Error &) {
        cudaGetLastError();
        std::printf("OOM on allocation (required %.2f MB)\n", theoretical_mb);
        results.push_back({s, -1, theoretical_mb, free_before / 1048576.0, -1, "OOM (Hardware VRAM Limit Exceeded)"});
        break;
      }
      if (random_inputs) { fill_normal(q, 0xDF03 + s); fill_normal(k, 0xDF13 + s); fill_normal(v, 0xDF23 + s); }
      const size_t free_after = df::get_memory_info().first;
      const double used_mb = free_before > free_after ? (free_before - free_after) / 1048576.0 : theoretical_mb;
      const int repeats = s <= 16384 ? 3 : 1;
      auto launch = [&]() {
        launch_fused_mha_forward(q.as_ptr(), k.as_ptr(), v.as_ptr(), out.as_mut_ptr(), (uint32_t)n_heads, (uint32_t)s,
                                 (uint32_t)d_head, scale, causal);
        df::check_status(df_attn_last_status(), "launch_fused_mha_forward");
      };
      if (s <= 16384) { launch(); df::cuda_sync(); }
      if (s <= max_timed) {
        std::vector<double> lat;
        for (int r = 0; r < repeats; ++r) {
          df::CudaEventTimer timer;
          timer.start();
          launch();
          lat.push_back(timer.stop_and_elapsed_ms());
        }
        df::cuda_sync();
        std::sort(lat.begin(), lat.end());
        const double median = lat[lat.size() / 2];
        const double tflops = 2.0 * n_heads * (double)s * (double)s * d_head / (median * 1e-3) / 1e12;
        std::printf("SUCCESS! Latency: %10.3f ms | VRAM: %9.2f MB | TFLOPs: %6.1f\n", median, used_mb, tflops);
        results.push_back({s, median, used_mb, free_after / 1048576.0, tflops, "SURVIVED (Online Softmax)"});
      } else {
        std::printf("SURVIVED! VRAM Allocated: %9.2f MB | Memory Scaling Verified (O(S) linear)\n", used_mb);
        results.push_back({s, -1, used_mb, free_after / 1048576.0, -1, "SURVIVED (Memory Scaling Verified)"});
      }
    }
    FILE *f = std::fopen(out_path.c_str(), "w");
    if (f) {
      std::fprintf(f, "{\n  \"metadata\": {\"device\": \"%s\", \"total_vram_mb\": %.2f, \"free_vram_mb\": %.2f, \"heads\": %zu, "
                      "\"d_head\": %zu, \"d_model\": %zu, \"causal\": true, \"precision\": \"Float32 API, TF32 tensor-core MMA\", "
                      "\"scope\": \"kernel_isolation\", \"inputs\": \"%s\", \"max_timed_seq\": %zu, "
                      "\"description\": \"Fused attention forward pass in isolation (Q, K, V, Out tensors only)\"},\n  \"results\": [\n",
                   prop.name, total_mb, free_mb, n_heads, d_head, d_model, random_inputs ? "seeded N(0,1)" : "zeros (as the reference)",
                   max_timed);
      for (size_t i = 0; i < results.size(); ++i) {
        const Result &r = results[i];
        std::fprintf(f, "    {\"seq_len\": %zu, \"latency_ms\": ", r.seq_len);
        if (r.latency_ms >= 0) std::fprintf(f, "%.6f", r.latency_ms); else std::fprintf(f, "null");
        std::fprintf(f, ", \"vram_allocated_mb\": %.2f, \"free_vram_mb\": %.2f, \"tflops\": ", r.vram_allocated_mb, r.free_vram_mb);
        if (r.tflops >= 0) std::fprintf(f, "%.3f", r.tflops); else std::fprintf(f, "null");
        std::fprintf(f, ", \"status\": \"%s\"}%s\n", r.status.c_str(), i + 1 < results.size() ? "," : "");
      }
      std::fprintf(f, "  ]\n}\n");
      std::fclose(f);
      std::printf("Saved results to %s\n", out_path.c_str());
    }
  } catch (const std::exception &e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}
