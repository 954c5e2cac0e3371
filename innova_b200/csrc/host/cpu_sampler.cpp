// Host-side token sampler: greedy arg-max, temperature, top-k, top-p and repetition penalty over a batch of logit rows.
//
// The reference samples on the CPU (src/sampler.cpp:12-122: arg-max, nth_element for top-k, a full sort for top-p, a
// penalty that divides positive and multiplies negative logits of tokens already generated). This is the same rule set for
// rows that live in host memory (CPU inference, the C API), written to agree with the device sampler of this package: the
// kept set is defined by value thresholds (every logit tied with the k-th largest, or with the last one inside the top-p
// mass, stays), and the token is drawn by inverse CDF in index order from one uniform number per row that the caller
// supplies. Given the same logits and uniforms the two samplers return the same tokens.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <thread>
#include <vector>

namespace {

int sample_row(const float* x_in, int V, float temperature, int top_k, float top_p, float u, const int32_t* hist, int T, float penalty,
               std::vector<float>& x, std::vector<float>& tmp) {
  x.assign(x_in, x_in + V);
  if (penalty != 1.0f && hist != nullptr && T > 0) {
    std::vector<int32_t> seen;
    seen.reserve(T);
    for (int t = 0; t < T; ++t)
      if (hist[t] >= 0 && hist[t] < V) seen.push_back(hist[t]);
    std::sort(seen.begin(), seen.end());
    seen.erase(std::unique(seen.begin(), seen.end()), seen.end());
    for (int32_t id : seen) x[id] = x[id] > 0.f ? x[id] / penalty : x[id] * penalty;
  }
  int arg = 0;
  for (int i = 1; i < V; ++i)
    if (x[i] > x[arg]) arg = i;  // the lowest index wins ties
  if (temperature <= 0.f || V == 1) return arg;
  const float inv_t = 1.f / temperature;
  for (int i = 0; i < V; ++i) x[i] *= inv_t;
  const float mx = x[arg];
  float thr = -INFINITY;
  if (top_k > 0 && top_k < V) {
    tmp.assign(x.begin(), x.end());
    std::nth_element(tmp.begin(), tmp.begin() + (top_k - 1), tmp.end(), [](float a, float b) { return a > b; });
    thr = tmp[top_k - 1];
  }
  if (top_p < 1.f) {
    tmp.clear();
    double total = 0.0;
    for (int i = 0; i < V; ++i)
      if (x[i] >= thr) {
        tmp.push_back(x[i]);
        total += std::exp((double)(x[i] - mx));
      }
    std::sort(tmp.begin(), tmp.end(), [](float a, float b) { return a > b; });
    double cum = 0.0;
    float last = tmp.empty() ? thr : tmp.front();
    for (float v : tmp) {  // the smallest prefix whose mass reaches top_p
      last = v;
      cum += std::exp((double)(v - mx));
      if (cum >= (double)top_p * total) break;
    }
    thr = std::max(thr, last);
  }
  double total = 0.0;
  for (int i = 0; i < V; ++i)
    if (x[i] >= thr) total += std::exp((double)(x[i] - mx));
  const double target = (double)std::min(std::max(u, 0.f), 0.99999994f) * total;
  double cum = 0.0;
  int lastkept = arg;
  for (int i = 0; i < V; ++i) {
    if (x[i] < thr) continue;
    cum += std::exp((double)(x[i] - mx));
    lastkept = i;
    if (cum > target) return i;
  }
  return lastkept;
}

}  // namespace

extern "C" {

// logits: B rows of V floats, row stride ld (elements). uniforms: B numbers in [0, 1) (ignored when temperature <= 0).
// history: B rows of T token ids (negative = unused) or null. Returns 0, or -1 for bad arguments.
int inv_cpu_sample(const float* logits, int B, int V, int ld, float temperature, int top_k, float top_p, const float* uniforms,
                   const int32_t* history, int T, float penalty, int32_t* out) {
  if (!logits || !out || B < 0 || V <= 0 || ld < V || (temperature > 0.f && !uniforms) || !(top_p > 0.f)) return -1;
  auto run = [&](int lo, int hi) {
    std::vector<float> x, tmp;
    for (int b = lo; b < hi; ++b)
      out[b] = sample_row(logits + (size_t)b * ld, V, temperature, top_k, top_p, uniforms ? uniforms[b] : 0.f,
                          history ? history + (size_t)b * T : nullptr, T, penalty, x, tmp);
  };
  unsigned workers = 1;
  if ((size_t)B * V >= (1u << 20) && B > 1) workers = std::min<unsigned>({(unsigned)B, std::max(1u, std::thread::hardware_concurrency()), 16u});
  if (workers <= 1) {
    run(0, B);
    return 0;
  }
  std::vector<std::thread> th;
  for (unsigned w = 0; w < workers; ++w) th.emplace_back(run, (int)((size_t)B * w / workers), (int)((size_t)B * (w + 1) / workers));
  for (auto& t : th) t.join();
  return 0;
}

}  // extern "C"
