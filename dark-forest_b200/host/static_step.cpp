// static_step.cpp — the attention calls of one static GPT-2 training step, made the way the reference's engine makes
// them, against a kernel library chosen at run time: an A/B harness for the drop-in claim.
//
// The reference's StaticGPT2 pre-allocates, per layer, q / k / v / attn_out of [seq_len, d_model]
// (darkforest-core/src/engine/static_gpt2.rs:365-379), one set of d_attn_out / d_q / d_k / d_v shared by all layers
// (:408-418) and one attention scratch of H*2*S*S floats shared through the contexts (:401-406); its forward calls
// attn_contexts[l].forward_device_into per layer (:1329-1336), its backward calls backward_device_into per layer
// in reverse (:1500-1510), and it synchronises once per step. This program does exactly that - through the legacy
// symbols launch_fused_mha_forward / launch_fused_mha_backward / darkforest_sync resolved with dlsym - for
//   --ours <libdarkforest_kernels.so>      this library
//   --ref  <libdf_reference_kernels.so>    the reference's own attention_fused.cu, compiled unmodified (optional)
// on the same seeded activations, times each backend with events on the legacy stream, compares the results of the
// two backends and prints one JSON line. It is a test and measurement harness: nothing of the product links it.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {

typedef void (*FwdFn)(const float *, const float *, const float *, float *, uint32_t, uint32_t, uint32_t, float, uint32_t);
typedef void (*BwdFn)(const float *, const float *, const float *, const float *, float *, float *, float *, float *, uint32_t,
                      uint32_t, uint32_t, float, uint32_t);
typedef void (*SyncFn)();

struct Backend {
  void *handle = nullptr;
  FwdFn fwd = nullptr;
  BwdFn bwd = nullptr;
  SyncFn sync = nullptr;  // the reference's attention file does not define darkforest_sync (matmul.cu does): may be null
  bool load(const char *path) {
    handle = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!handle) {
      fprintf(stderr, "dlopen %s: %s\n", path, dlerror());
      return false;
    }
    fwd = (FwdFn)dlsym(handle, "launch_fused_mha_forward");
    bwd = (BwdFn)dlsym(handle, "launch_fused_mha_backward");
    sync = (SyncFn)dlsym(handle, "darkforest_sync");
    return fwd && bwd;
  }
};

#define CK(x)                                                                                 \
  do {                                                                                        \
    cudaError_t e__ = (x);                                                                    \
    if (e__ != cudaSuccess) {                                                                 \
      fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e__), __FILE__, __LINE__); \
      exit(2);                                                                                \
    }                                                                                         \
  } while (0)

// splitmix64 -> approximately N(0,1) (sum of four uniforms, variance-normalised): cheap, seeded, same on every run
__global__ void k_fill(float *dst, size_t n, uint64_t seed) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (i + 1);
    float acc = 0.f;
    for (int r = 0; r < 4; ++r) {
      z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
      z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
      z = z ^ (z >> 31);
      acc += (float)(z >> 40) * (1.0f / 16777216.0f) - 0.5f;
    }
    dst[i] = acc * 1.7320508f;  // var(sum of 4 U(-.5,.5)) = 1/3
  }
}

struct Step {
  int layers, heads;
  uint32_t seq, d_head;
  size_t n;
  std::vector<float *> q, k, v, attn_out;
  float *d_attn_out = nullptr, *d_q = nullptr, *d_k = nullptr, *d_v = nullptr, *prob = nullptr;
  void alloc(int L, int H, uint32_t S, uint32_t D) {
    layers = L; heads = H; seq = S; d_head = D;
    n = (size_t)S * H * D;
    for (int l = 0; l < L; ++l) {
      float *p[4];
      for (auto &x : p) CK(cudaMalloc(&x, n * 4));
      q.push_back(p[0]); k.push_back(p[1]); v.push_back(p[2]); attn_out.push_back(p[3]);
      k_fill<<<296, 256>>>(p[0], n, 1000 + 10 * l);
      k_fill<<<296, 256>>>(p[1], n, 1001 + 10 * l);
      k_fill<<<296, 256>>>(p[2], n, 1002 + 10 * l);
    }
    for (float **x : {&d_attn_out, &d_q, &d_k, &d_v}) CK(cudaMalloc(x, n * 4));
    k_fill<<<296, 256>>>(d_attn_out, n, 77);
    CK(cudaMalloc(&prob, (size_t)H * 2 * S * S * 4));  // lib.rs:2019-2027
    CK(cudaDeviceSynchronize());
  }
};

struct Timing { float fwd_ms = 0, bwd_ms = 0; };

Timing run(const Backend &b, Step &st, int steps, int warmup) {
  const float scale = 1.0f / sqrtf((float)st.d_head);  // static_gpt2.rs:1291
  cudaEvent_t e0, e1, e2;
  CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1)); CK(cudaEventCreate(&e2));
  Timing t;
  for (int it = 0; it < warmup + steps; ++it) {
    CK(cudaEventRecord(e0, 0));
    for (int l = 0; l < st.layers; ++l)
      b.fwd(st.q[l], st.k[l], st.v[l], st.attn_out[l], st.heads, st.seq, st.d_head, scale, 1);
    CK(cudaEventRecord(e1, 0));
    for (int l = st.layers - 1; l >= 0; --l)
      b.bwd(st.q[l], st.k[l], st.v[l], st.d_attn_out, st.d_q, st.d_k, st.d_v, st.prob, st.heads, st.seq, st.d_head, scale, 1);
    CK(cudaEventRecord(e2, 0));
    if (b.sync) b.sync();  // the one synchronisation per step (kernels.rs:6-8)
    CK(cudaDeviceSynchronize());
    if (it >= warmup) {
      float a = 0, c = 0;
      CK(cudaEventElapsedTime(&a, e0, e1));
      CK(cudaEventElapsedTime(&c, e1, e2));
      t.fwd_ms += a / steps;
      t.bwd_ms += c / steps;
    }
  }
  return t;
}

std::vector<float> fetch(const float *d, size_t n) {
  std::vector<float> h(n);
  CK(cudaMemcpy(h.data(), d, n * 4, cudaMemcpyDeviceToHost));
  return h;
}
double max_abs(const std::vector<float> &a) {
  double m = 0;
  for (float x : a) m = fmax(m, fabs((double)x));
  return m;
}
double max_diff(const std::vector<float> &a, const std::vector<float> &b) {
  double m = 0;
  for (size_t i = 0; i < a.size(); ++i) m = fmax(m, fabs((double)a[i] - (double)b[i]));
  return m;
}

}  // namespace

int main(int argc, char **argv) {
  const char *ours = nullptr, *ref = nullptr;
  int layers = 12, heads = 12, steps = 3, warmup = 1;
  uint32_t seq = 4096, d_head = 64;
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string a = argv[i];
    if (a == "--ours") ours = argv[i + 1];
    else if (a == "--ref") ref = argv[i + 1];
    else if (a == "--layers") layers = atoi(argv[i + 1]);
    else if (a == "--heads") heads = atoi(argv[i + 1]);
    else if (a == "--seq") seq = (uint32_t)atoi(argv[i + 1]);
    else if (a == "--dhead") d_head = (uint32_t)atoi(argv[i + 1]);
    else if (a == "--steps") steps = atoi(argv[i + 1]);
    else if (a == "--warmup") warmup = atoi(argv[i + 1]);
  }
  if (!ours) {
    fprintf(stderr, "usage: static_step --ours <lib.so> [--ref <lib.so>] [--layers 12 --heads 12 --seq 4096 --dhead 64 --steps 3]\n");
    return 1;
  }
  Backend bo, br;
  if (!bo.load(ours)) return 1;
  const bool have_ref = ref && br.load(ref);
  Step st;
  st.alloc(layers, heads, seq, d_head);
  const Timing to = run(bo, st, steps, warmup);
  // results of the step's last calls: attn_out of the last layer, gradients of layer 0 (the shared buffers)
  const std::vector<float> o_ours = fetch(st.attn_out[layers - 1], st.n), dq_ours = fetch(st.d_q, st.n), dk_ours = fetch(st.d_k, st.n),
                           dv_ours = fetch(st.d_v, st.n);
  const double fwd_flop = 2.0 * heads * (double)seq * seq * d_head * layers;  // causal accounting, per step
  printf("{\"layers\": %d, \"heads\": %d, \"seq\": %u, \"d_head\": %u, \"steps\": %d, \"ours\": {\"fwd_ms\": %.4f, \"bwd_ms\": %.4f, "
         "\"fwd_bwd_tflops_2.5x\": %.2f}",
         layers, heads, seq, d_head, steps, to.fwd_ms, to.bwd_ms, 2.5 * fwd_flop / ((to.fwd_ms + to.bwd_ms) * 1e-3) / 1e12);
  if (have_ref) {
    const Timing tr = run(br, st, steps > 2 ? 2 : steps, 1);
    const std::vector<float> o_ref = fetch(st.attn_out[layers - 1], st.n), dq_ref = fetch(st.d_q, st.n), dk_ref = fetch(st.d_k, st.n),
                             dv_ref = fetch(st.d_v, st.n);
    auto rel = [&](const std::vector<float> &a, const std::vector<float> &b) { return max_diff(a, b) / fmax(max_abs(b), 0.25); };
    printf(", \"reference\": {\"fwd_ms\": %.4f, \"bwd_ms\": %.4f, \"fwd_bwd_tflops_2.5x\": %.3f}, \"speedup_fwd\": %.1f, "
           "\"speedup_bwd\": %.1f, \"speedup_step\": %.1f, \"max_abs_diff_attn_out\": %.3e, \"max_rel_diff_dq\": %.3e, "
           "\"max_rel_diff_dk\": %.3e, \"max_rel_diff_dv\": %.3e",
           tr.fwd_ms, tr.bwd_ms, 2.5 * fwd_flop / ((tr.fwd_ms + tr.bwd_ms) * 1e-3) / 1e12, tr.fwd_ms / to.fwd_ms, tr.bwd_ms / to.bwd_ms,
           (tr.fwd_ms + tr.bwd_ms) / (to.fwd_ms + to.bwd_ms), max_diff(o_ours, o_ref), rel(dq_ours, dq_ref), rel(dk_ours, dk_ref),
           rel(dv_ours, dv_ref));
  }
  printf("}\n");
  return 0;
}
