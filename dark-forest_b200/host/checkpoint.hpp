// checkpoint.hpp — the reference's StaticGPT2 checkpoint file in C++, read and written bit for bit
// (darkforest-core/src/engine/static_gpt2.rs:1924-2006 save_checkpoint, :2012-2114 load_checkpoint).
//
// Little endian throughout. One block per tensor: u64 element count, then that many f32. Weights first
// (tok_emb, pos_emb, ln_f_gamma, ln_f_beta, lm_head, then per layer ln1_gamma, ln1_beta, wq, bq, wk, bk, wv, bv, wo,
// bo, ln2_gamma, ln2_beta, w1, b1, w2, b2), then the AdamW moments in the same order as (m, v) block pairs, then a
// footer: u64 step_count and f32 lr, beta1, beta2, eps, wd. No shapes are stored: the reader knows the model's
// configuration and reports the reference's "tensor size mismatch: file=.. model=.." when a block disagrees.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace df {

struct Gpt2Config {
  size_t vocab_size, d_model, n_heads, n_layers, d_ff, seq_len;
};

struct Gpt2Checkpoint {
  std::vector<std::string> names;            // file order
  std::vector<std::vector<float>> weights;   // one per name
  std::vector<std::vector<float>> m, v;      // AdamW moments, one pair per name
  uint64_t step_count = 0;
  float lr = 3e-4f, beta1 = 0.9f, beta2 = 0.95f, eps = 1e-8f, wd = 0.1f;
};

inline size_t checkpoint_numel(const Gpt2Config &c, const std::string &name) {
  const std::string base = name.substr(name.rfind('.') == std::string::npos ? 0 : name.rfind('.') + 1);
  const size_t d = c.d_model, f = c.d_ff;
  if (base == "tok_emb" || base == "lm_head") return c.vocab_size * d;
  if (base == "pos_emb") return c.seq_len * d;
  if (base == "wq" || base == "wk" || base == "wv" || base == "wo") return d * d;
  if (base == "w1" || base == "w2") return d * f;
  if (base == "b1") return f;
  return d;  // layer-norm gains and shifts, bq, bk, bv, bo, b2
}

inline std::vector<std::string> checkpoint_tensor_names(const Gpt2Config &c) {
  std::vector<std::string> n = {"tok_emb", "pos_emb", "ln_f_gamma", "ln_f_beta", "lm_head"};
  static const char *per_layer[] = {"ln1_gamma", "ln1_beta", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "ln2_gamma", "ln2_beta",
                                    "w1", "b1", "w2", "b2"};
  for (size_t l = 0; l < c.n_layers; ++l)
    for (const char *p : per_layer) n.push_back("layers." + std::to_string(l) + "." + p);
  return n;
}

namespace detail {
inline void put_u64(FILE *f, uint64_t x) {
  unsigned char b[8];
  for (int i = 0; i < 8; ++i) b[i] = (unsigned char)(x >> (8 * i));
  if (fwrite(b, 1, 8, f) != 8) throw std::runtime_error("save_checkpoint: write failed");
}
inline void put_f32s(FILE *f, const float *p, size_t n) {
  // the build targets little-endian hosts (x86-64, aarch64): f32 words go out as they are
  if (n && fwrite(p, 4, n, f) != n) throw std::runtime_error("save_checkpoint: write failed");
}
inline uint64_t get_u64(FILE *f) {
  unsigned char b[8];
  if (fread(b, 1, 8, f) != 8) throw std::runtime_error("load_checkpoint: failed to fill whole buffer");
  uint64_t x = 0;
  for (int i = 0; i < 8; ++i) x |= (uint64_t)b[i] << (8 * i);
  return x;
}
inline std::vector<float> get_block(FILE *f, size_t want) {
  const uint64_t n = get_u64(f);
  if (n != want)
    throw std::runtime_error("load_checkpoint: tensor size mismatch: file=" + std::to_string(n) + " model=" + std::to_string(want));
  std::vector<float> d(n);
  if (n && fread(d.data(), 4, n, f) != n) throw std::runtime_error("load_checkpoint: failed to fill whole buffer");
  return d;
}
}  // namespace detail

inline void save_checkpoint(const std::string &path, const Gpt2Config &c, const Gpt2Checkpoint &ck) {
  FILE *f = fopen(path.c_str(), "wb");
  if (!f) throw std::runtime_error("save_checkpoint: cannot create " + path);
  try {
    const std::vector<std::string> names = checkpoint_tensor_names(c);
    if (ck.weights.size() != names.size() || ck.m.size() != names.size() || ck.v.size() != names.size())
      throw std::runtime_error("save_checkpoint: tensor count does not match the configuration");
    for (size_t i = 0; i < names.size(); ++i) {
      if (ck.weights[i].size() != checkpoint_numel(c, names[i])) throw std::runtime_error("save_checkpoint: size of " + names[i]);
      detail::put_u64(f, ck.weights[i].size());
      detail::put_f32s(f, ck.weights[i].data(), ck.weights[i].size());
    }
    for (size_t i = 0; i < names.size(); ++i) {
      if (ck.m[i].size() != ck.weights[i].size() || ck.v[i].size() != ck.weights[i].size())
        throw std::runtime_error("save_checkpoint: moments of " + names[i]);
      detail::put_u64(f, ck.m[i].size());
      detail::put_f32s(f, ck.m[i].data(), ck.m[i].size());
      detail::put_u64(f, ck.v[i].size());
      detail::put_f32s(f, ck.v[i].data(), ck.v[i].size());
    }
    detail::put_u64(f, ck.step_count);
    const float foot[5] = {ck.lr, ck.beta1, ck.beta2, ck.eps, ck.wd};
    detail::put_f32s(f, foot, 5);
  } catch (...) {
    fclose(f);
    throw;
  }
  fclose(f);
}

inline Gpt2Checkpoint load_checkpoint(const std::string &path, const Gpt2Config &c) {
  FILE *f = fopen(path.c_str(), "rb");
  if (!f) throw std::runtime_error("load_checkpoint: cannot open " + path);
  Gpt2Checkpoint ck;
  try {
    ck.names = checkpoint_tensor_names(c);
    for (const std::string &n : ck.names) ck.weights.push_back(detail::get_block(f, checkpoint_numel(c, n)));
    for (const std::string &n : ck.names) {
      ck.m.push_back(detail::get_block(f, checkpoint_numel(c, n)));
      ck.v.push_back(detail::get_block(f, checkpoint_numel(c, n)));
    }
    ck.step_count = detail::get_u64(f);
    float foot[5];
    if (fread(foot, 4, 5, f) != 5) throw std::runtime_error("load_checkpoint: failed to fill whole buffer");
    ck.lr = foot[0]; ck.beta1 = foot[1]; ck.beta2 = foot[2]; ck.eps = foot[3]; ck.wd = foot[4];
  } catch (...) {
    fclose(f);
    throw;
  }
  fclose(f);
  return ck;
}

}  // namespace df
