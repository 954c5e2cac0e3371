// Format registry, quality measurement, format selection under a bits-per-weight target, the
// adaptive hard-budget mix allocator and the importance-tiered planner.
//
// Behaviour follows the reference's FormatRegistry (src/format_registry.cpp:17-101 descriptors and
// mixes, :39-70 measured est_mse with mt19937(20260803), :231-387 selection that never exceeds the
// target, :477-599 greedy benefit-per-byte allocation under a hard byte budget) and FormatPlanner
// (src/format_planner.cpp:12-122 importance scoring and tiered allocation, :133-315 interpolated
// two-format plans). Everything is measured through the canonical block codec of oil_codec.cpp.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <queue>
#include <random>
#include <string>
#include <vector>

#include "oil_codec.h"

namespace inv {

struct Mix {
  const char* name;
  int ntiers;
  int fmt[4];
  float frac[4];
  float bpw;      // effective bits per weight: a hard cap for the allocator
  bool adaptive;
};

static const Mix kMixes[] = {
    {"OIL8+OIL2_1_99", 2, {OIL8, OIL2, 0, 0}, {0.01f, 0.99f, 0, 0}, 2.06f, false},
    {"OIL8+OIL4_5_95", 2, {OIL8, OIL4, 0, 0}, {0.05f, 0.95f, 0, 0}, 4.20f, false},
    {"OIL4+OIL2_10_90", 2, {OIL4, OIL2, 0, 0}, {0.10f, 0.90f, 0, 0}, 2.20f, false},
    {"OIL8+OIL2_10_90", 2, {OIL8, OIL2, 0, 0}, {0.10f, 0.90f, 0, 0}, 2.60f, false},
    {"SPARK+OIL8_5_95", 2, {SPARK_Q0, OIL8, 0, 0}, {0.05f, 0.95f, 0, 0}, 7.675f, false},
    {"OIL16+OIL4_1_99", 2, {OIL16, OIL4, 0, 0}, {0.01f, 0.99f, 0, 0}, 4.12f, false},
    {"OIL16+OIL8_5_95", 2, {OIL16, OIL8, 0, 0}, {0.05f, 0.95f, 0, 0}, 8.40f, false},
    {"OIL32+OIL8_1_99", 2, {OIL32, OIL8, 0, 0}, {0.01f, 0.99f, 0, 0}, 8.24f, false},
    {"SPARK_MIX_Q0", 4, {OIL8_GRP, OIL4_GRP, OIL2_GRP, OIL1_GRP}, {0.01f, 0.02f, 0.52f, 0.45f}, 1.925f, true},
    {"QUAD_OIL2_OIL4_OIL8_OIL16", 4, {OIL16, OIL8, OIL4, OIL2}, {0.01f, 0.05f, 0.24f, 0.70f}, 2.92f, false},
    {"QUAD_OIL4_OIL8_OIL16_OIL32", 4, {OIL32, OIL16, OIL8, OIL4}, {0.01f, 0.05f, 0.24f, 0.70f}, 5.84f, false},
    {"QUAD_SPARK_Q1", 4, {OIL32, OIL8_GRP, OIL2_GRP, OIL1_GRP}, {0.01f, 0.01f, 0.46f, 0.52f}, 2.075f, true},
};
constexpr int kNumMixes = sizeof(kMixes) / sizeof(kMixes[0]);

// Sum of squared error and stored bytes of one block through the codec.
static void block_cost(int fmt, const float* w, int n, double* sse, size_t* bytes) {
  std::vector<uint8_t> idx, cb;
  std::vector<float> dq((size_t)n);
  encode_block(fmt, w, n, idx, cb);
  decode_block(fmt, idx.data(), idx.size(), cb.data(), cb.size(), (uint32_t)n, dq.data());
  double s = 0.0;
  for (int i = 0; i < n; ++i) {
    const double d = (double)w[i] - dq[(size_t)i];
    s += d * d;
  }
  *sse = s;
  *bytes = idx.size() + cb.size();
}

static float measure_mse(int fmt, const float* d, int64_t n, int block) {
  double total = 0.0;
  for (int64_t lo = 0; lo < n; lo += block) {
    double sse;
    size_t by;
    block_cost(fmt, d + lo, (int)std::min<int64_t>(block, n - lo), &sse, &by);
    total += sse;
  }
  return (float)(total / (double)n);
}

// Worst MSE over three fixed unit-scale distributions (Gaussian, uniform [-2, 2], Laplace).
static const float* est_mse_table() {
  static float table[FORMAT_COUNT];
  static std::once_flag once;
  std::call_once(once, []() {
    const int64_t n = 16384;
    std::vector<float> g((size_t)n), u((size_t)n), l((size_t)n);
    std::mt19937 rng(20260803);
    std::normal_distribution<float> gd(0.0f, 1.0f);
    std::uniform_real_distribution<float> ud(-2.0f, 2.0f);
    std::exponential_distribution<float> ed(1.0f);
    for (int64_t i = 0; i < n; ++i) {
      g[(size_t)i] = gd(rng);
      u[(size_t)i] = ud(rng);
      l[(size_t)i] = ed(rng) - ed(rng);
    }
    for (int f = 0; f < FORMAT_COUNT; ++f) {
      if (f == OIL32) {
        table[f] = 0.0f;
        continue;
      }
      float worst = 0.0f;
      for (const std::vector<float>* d : {&g, &u, &l}) worst = std::max(worst, measure_mse(f, d->data(), n, 256));
      table[f] = worst;
    }
  });
  return table;
}

struct BlockPlan {
  std::vector<uint8_t> formats;
  int64_t bytes = 0;
  double sse = 0.0;
};

// Every block starts on the cheapest member of the mix; a max-heap ordered by error reduction per
// extra byte upgrades blocks one step at a time while the total stays within ceil(bpw * n / 8).
static BlockPlan allocate_mix(const Mix& mix, const float* data, int64_t n, int block) {
  BlockPlan plan;
  std::vector<int> ladder(mix.fmt, mix.fmt + mix.ntiers);
  std::sort(ladder.begin(), ladder.end(), [](int a, int b) { return format_bpw(a) < format_bpw(b); });
  ladder.erase(std::unique(ladder.begin(), ladder.end()), ladder.end());
  const int T = (int)ladder.size();
  const int64_t nb = (n + block - 1) / block;
  const int64_t budget = (int64_t)std::ceil((double)mix.bpw * (double)n / 8.0);
  std::vector<double> sse((size_t)nb * T);
  std::vector<size_t> bytes((size_t)nb * T);
  for (int64_t b = 0; b < nb; ++b) {
    const int cnt = (int)std::min<int64_t>(block, n - b * block);
    for (int t = 0; t < T; ++t) block_cost(ladder[(size_t)t], data + b * block, cnt, &sse[(size_t)b * T + t], &bytes[(size_t)b * T + t]);
  }
  std::vector<int> tier((size_t)nb, 0);
  int64_t used = 0;
  for (int64_t b = 0; b < nb; ++b) used += (int64_t)bytes[(size_t)b * T];
  struct Cand {
    double gain;
    int64_t b;
    int to;
    bool operator<(const Cand& o) const { return gain < o.gain; }
  };
  std::priority_queue<Cand> heap;
  auto push = [&](int64_t b) {
    const int t = tier[(size_t)b];
    if (t + 1 >= T) return;
    const double ds = sse[(size_t)b * T + t] - sse[(size_t)b * T + t + 1];
    const double db = (double)bytes[(size_t)b * T + t + 1] - (double)bytes[(size_t)b * T + t];
    if (ds <= 0.0) return;
    heap.push({db <= 0.0 ? 1e300 : ds / db, b, t + 1});
  };
  for (int64_t b = 0; b < nb; ++b) push(b);
  while (!heap.empty()) {
    const Cand c = heap.top();
    heap.pop();
    if (tier[(size_t)c.b] + 1 != c.to) continue;
    const int64_t extra = (int64_t)bytes[(size_t)c.b * T + c.to] - (int64_t)bytes[(size_t)c.b * T + c.to - 1];
    if (used + extra > budget) continue;  // a cheaper upgrade elsewhere may still fit
    used += extra;
    tier[(size_t)c.b] = c.to;
    push(c.b);
  }
  plan.formats.resize((size_t)nb);
  for (int64_t b = 0; b < nb; ++b) {
    plan.formats[(size_t)b] = (uint8_t)ladder[(size_t)tier[(size_t)b]];
    plan.sse += sse[(size_t)b * T + tier[(size_t)b]];
  }
  plan.bytes = used;
  return plan;
}

}  // namespace inv

using namespace inv;

extern "C" {

int reg_num_singles() { return FORMAT_COUNT; }
float reg_est_mse(int fmt) { return (fmt >= 0 && fmt < FORMAT_COUNT) ? est_mse_table()[fmt] : 1.0f; }
int reg_num_mixes() { return kNumMixes; }
// name_out: at least 64 bytes. fmts / fracs: 4 entries.
int reg_mix_info(int i, char* name_out, float* bpw, int* ntiers, int* fmts, float* fracs, int* adaptive) {
  if (i < 0 || i >= kNumMixes) return -1;
  std::strncpy(name_out, kMixes[i].name, 63);
  name_out[63] = 0;
  *bpw = kMixes[i].bpw;
  *ntiers = kMixes[i].ntiers;
  for (int t = 0; t < 4; ++t) {
    fmts[t] = kMixes[i].fmt[t];
    fracs[t] = kMixes[i].frac[t];
  }
  *adaptive = kMixes[i].adaptive ? 1 : 0;
  return 0;
}
float reg_measure_mse(int fmt, const float* d, int64_t n, int block) { return measure_mse(fmt, d, n, block > 0 ? block : 256); }

// Lowest-error single format whose claimed bpw does not exceed the target (measured on `d` when given,
// else by the registry's estimate). Returns the wire format id.
int reg_select_best_format(float target_bpw, const float* d, int64_t n) {
  int best = -1;
  float best_mse = 1e30f;
  for (int f = 0; f < FORMAT_COUNT; ++f) {
    if (format_bpw(f) > target_bpw + 1e-6f) continue;
    const float mse = (d && n > 0) ? measure_mse(f, d, n, 256) : est_mse_table()[f];
    if (mse < best_mse) {
      best_mse = mse;
      best = f;
    }
  }
  if (best < 0) best = OIL1;  // nothing fits: the cheapest format
  return best;
}

// Allocates the blocks of `d` over the members of mix `i` under its byte budget. Returns the number of
// blocks written to fmts_out; *bytes_out = payload bytes, *mse_out = resulting mean squared error.
int64_t reg_allocate_mix(int i, const float* d, int64_t n, int block, uint8_t* fmts_out, int64_t* bytes_out, float* mse_out) {
  if (i < 0 || i >= kNumMixes || !d || n <= 0) return -1;
  BlockPlan p = allocate_mix(kMixes[i], d, n, block > 0 ? block : 256);
  std::memcpy(fmts_out, p.formats.data(), p.formats.size());
  if (bytes_out) *bytes_out = p.bytes;
  if (mse_out) *mse_out = (float)(p.sse / (double)n);
  return (int64_t)p.formats.size();
}

// Best mix at or under the target by measured error; -1 if no mix fits.
int reg_select_best_mix(float target_bpw, const float* d, int64_t n) {
  int best = -1;
  double best_sse = 1e300;
  for (int i = 0; i < kNumMixes; ++i) {
    if (kMixes[i].bpw > target_bpw + 1e-6f) continue;
    if (!d || n <= 0) {
      if (best < 0 || kMixes[i].bpw > kMixes[best].bpw) best = i;
      continue;
    }
    BlockPlan p = allocate_mix(kMixes[i], d, n, 256);
    if (p.sse < best_sse) {
      best_sse = p.sse;
      best = i;
    }
  }
  return best;
}

// Planner: per-block formats for a tensor under a target bpw. Two neighbouring single formats (the best
// at or under the target and the next more precise one) are interpolated: the most important blocks
// get the precise one, as many as the byte budget ceil(target * n / 8) allows. importance: one value
// per block (null: mean |w| of the block). Returns the number of blocks.
int64_t reg_plan_tensor(float target_bpw, const float* d, int64_t n, int block, const float* importance, uint8_t* fmts_out,
                        int64_t* bytes_out) {
  if (!d || n <= 0) return -1;
  if (block <= 0) block = 256;
  const int64_t nb = (n + block - 1) / block;
  const int lo = reg_select_best_format(target_bpw, d, std::min<int64_t>(n, 65536));
  int hi = -1;
  float hi_mse = 1e30f;
  for (int f = 0; f < FORMAT_COUNT; ++f) {  // the cheapest format that is more precise than `lo`
    if (format_bpw(f) <= format_bpw(lo) + 1e-6f) continue;
    if (est_mse_table()[f] >= est_mse_table()[lo]) continue;
    if (hi < 0 || format_bpw(f) < format_bpw(hi) || (format_bpw(f) == format_bpw(hi) && est_mse_table()[f] < hi_mse)) {
      hi = f;
      hi_mse = est_mse_table()[f];
    }
  }
  std::vector<float> imp((size_t)nb);
  for (int64_t b = 0; b < nb; ++b) {
    if (importance) {
      imp[(size_t)b] = importance[b];
    } else {
      const int cnt = (int)std::min<int64_t>(block, n - b * block);
      double s = 0.0;
      for (int i = 0; i < cnt; ++i) s += std::fabs(d[b * block + i]);
      imp[(size_t)b] = (float)(s / cnt);
    }
  }
  std::vector<int64_t> order((size_t)nb);
  for (int64_t b = 0; b < nb; ++b) order[(size_t)b] = b;
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return imp[(size_t)a] > imp[(size_t)b]; });
  const int64_t budget = (int64_t)std::ceil((double)target_bpw * (double)n / 8.0);
  int64_t used = 0;
  for (int64_t b = 0; b < nb; ++b) {
    fmts_out[b] = (uint8_t)lo;
    used += (int64_t)claimed_bytes(lo, (uint32_t)std::min<int64_t>(block, n - b * block)) + 1;
  }
  if (hi >= 0) {
    for (int64_t k = 0; k < nb; ++k) {
      const int64_t b = order[(size_t)k];
      const uint32_t cnt = (uint32_t)std::min<int64_t>(block, n - b * block);
      const int64_t extra = (int64_t)claimed_bytes(hi, cnt) - (int64_t)claimed_bytes(lo, cnt);
      if (used + extra > budget) break;
      used += extra;
      fmts_out[b] = (uint8_t)hi;
    }
  }
  if (bytes_out) *bytes_out = used;
  return nb;
}

}  // extern "C"
