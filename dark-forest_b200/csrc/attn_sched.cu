// attn_sched.cu — host side of the explicit work lists of the persistent kernels: a MULTIFIT
// assignment of weighted items to CTAs, cached per shape. Nothing here touches the GPU.
#include <algorithm>
#include <mutex>
#include <numeric>
#include <vector>

#include "df_common.cuh"

namespace df {
namespace {

struct Entry {
  SchedKey key;
  int n_items;
  SchedTable table;
  bool valid = false;
};
constexpr int kEntries = 16;
Entry g_cache[kEntries];
int g_next = 0;
std::mutex g_mutex;

bool same(const SchedKey &a, const SchedKey &b) {
  return a.kind == b.kind && a.bh == b.bh && a.sq == b.sq && a.sk == b.sk && a.causal == b.causal && a.shift == b.shift &&
         a.grid == b.grid;
}

// First-fit decreasing under capacity `cap`: bin_of[i] for the items in `order`; false if one does not fit.
bool first_fit(const std::vector<uint32_t> &w, const std::vector<int> &order, int grid, uint64_t cap, std::vector<int> *bin_of) {
  std::vector<uint64_t> load(grid, 0);
  for (int i : order) {
    int b = 0;
    while (b < grid && load[b] + w[i] > cap) ++b;
    if (b == grid) return false;
    load[b] += w[i];
    (*bin_of)[i] = b;
  }
  return true;
}

void build(const std::vector<uint32_t> &w, int grid, SchedTable *out) {
  const int n = (int)w.size();
  out->used = 0;
  if (n <= grid || n > kSchedMaxItems || grid > kSchedMaxCtas) return;
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return w[a] > w[b]; });
  const uint64_t total = std::accumulate(w.begin(), w.end(), (uint64_t)0);
  uint64_t lo = std::max<uint64_t>(w[order[0]], (total + grid - 1) / grid);
  // the snake order's heaviest CTA is the value to beat
  std::vector<uint64_t> snake(grid, 0);
  for (int k = 0; k < n; ++k) {
    const int r = k / grid, c = (r & 1) ? grid - 1 - k % grid : k % grid;
    snake[c] += w[order[k]];
  }
  uint64_t hi = *std::max_element(snake.begin(), snake.end());
  std::vector<int> best, trial(n);
  while (lo < hi) {
    const uint64_t mid = (lo + hi) / 2;
    if (first_fit(w, order, grid, mid, &trial)) {
      best = trial;
      hi = mid;
    } else {
      lo = mid + 1;
    }
  }
  if (best.empty()) return;  // nothing below the snake order's makespan is feasible for first-fit
  std::vector<int> count(grid + 1, 0);
  for (int i = 0; i < n; ++i) ++count[best[i] + 1];
  for (int c = 0; c < grid; ++c) count[c + 1] += count[c];
  for (int c = 0; c <= grid; ++c) out->off[c] = (uint16_t)count[c];
  std::vector<int> fill(count.begin(), count.end() - 1);
  for (int i : order) out->items[fill[best[i]]++] = (uint16_t)i;  // heaviest first within a CTA
  out->used = 1;
}

}  // namespace

void schedule_for(const SchedKey &key, int n_items, uint32_t (*weight)(const void *ctx, int item), const void *ctx,
                  SchedTable *out) {
  out->used = 0;
  if (n_items <= key.grid || n_items > kSchedMaxItems || key.grid > kSchedMaxCtas || !key.causal) return;
  if (option(DF_OPT_SCHED_TABLE) == 0) return;
  std::lock_guard<std::mutex> guard(g_mutex);
  for (const Entry &e : g_cache)
    if (e.valid && e.n_items == n_items && same(e.key, key)) {
      *out = e.table;
      return;
    }
  std::vector<uint32_t> w(n_items);
  for (int i = 0; i < n_items; ++i) w[i] = weight(ctx, i);
  Entry &e = g_cache[g_next];
  g_next = (g_next + 1) % kEntries;
  e.key = key;
  e.n_items = n_items;
  build(w, key.grid, &e.table);
  e.valid = true;
  *out = e.table;
}

}  // namespace df

// Host-only probe of the builder (tests): the work lists for `n` items of the given weights on `grid`
// CTAs. Returns 1 and fills off[grid + 1], items[n] when a table is produced, 0 when the launchers
// would fall back to the snake order.
extern "C" int df_attn_schedule_build(const uint32_t *weights, int n, int grid, uint16_t *off, uint16_t *items) {
  if (!weights || !off || !items || n <= 0 || grid <= 0) return 0;
  static thread_local df::SchedTable t;
  df::build(std::vector<uint32_t>(weights, weights + n), grid, &t);
  if (!t.used) return 0;
  for (int c = 0; c <= grid; ++c) off[c] = t.off[c];
  for (int i = 0; i < n; ++i) items[i] = t.items[i];
  return 1;
}

