// checkpoint_tool — reads a StaticGPT2 checkpoint with the C++ reader and writes it back with the C++ writer
// (host only, no GPU): the round trip the tests compare byte for byte with the Python implementation.
// usage: checkpoint_tool <in> <out> <vocab> <d_model> <n_heads> <n_layers> <d_ff> <seq_len>
#include <cstdio>
#include <cstdlib>

#include "checkpoint.hpp"

int main(int argc, char **argv) {
  if (argc != 9) {
    fprintf(stderr, "usage: checkpoint_tool <in> <out> <vocab> <d_model> <n_heads> <n_layers> <d_ff> <seq_len>\n");
    return 2;
  }
  df::Gpt2Config c{(size_t)atoll(argv[3]), (size_t)atoll(argv[4]), (size_t)atoll(argv[5]), (size_t)atoll(argv[6]), (size_t)atoll(argv[7]),
                   (size_t)atoll(argv[8])};
  try {
    const df::Gpt2Checkpoint ck = df::load_checkpoint(argv[1], c);
    df::save_checkpoint(argv[2], c, ck);
    double sum = 0;
    for (const auto &w : ck.weights)
      for (float x : w) sum += x;
    printf("{\"tensors\": %zu, \"step_count\": %llu, \"lr\": %g, \"weight_sum\": %.9g}\n", ck.weights.size(),
           (unsigned long long)ck.step_count, ck.lr, sum);
  } catch (const std::exception &e) {
    fprintf(stderr, "%s\n", e.what());
    return 1;
  }
  return 0;
}
