// Speculative-decoding verification for a batch of sequences in one launch.
//
// Replaces the accept / reject / resample loop of SpeculativeDecoder::generate and verify_tokens
// (src/inference_opt.cpp:131-281) and the exact-match SmallBatchVerifier
// (src/speculative_decoder.cpp:184-236).
//
// Inputs per sequence b: G draft tokens, the target model's logits for the G draft positions plus one
// bonus position ([B, G+1, V] fp32), and either the draft model's logits ([B, G, V]) or nothing (the
// reference's draft-free mode uses p_draft = 1/V). One CTA walks its sequence's positions in order:
//   mode 0 (rejection sampling): accept token t_i with probability min(1, p_target(t_i)/(p_draft(t_i)+1e-10));
//       at the first rejection draw the replacement from normalise(max(0, p_target - p_draft)) (from
//       p_target itself if that residual is empty); if every draft survives, draw the bonus token from
//       the target's distribution at position G.
//   mode 1 (exact match): accept while argmax(target_i) == t_i; the replacement / bonus token is the
//       target's argmax at the first mismatch / at position G.
// Uniform numbers come from the host generator: uniforms[b, 0..G-1] decide acceptance, uniforms[b, G]
// drives the draw. Output: n_accept[b] in [0, G], next_token[b]. The walk stops at the first
// rejection, so the cost is proportional to the accepted prefix. Temperature divides both logit sets.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {
namespace sv {

constexpr int THREADS = 512;

struct RowStat {
  float mx, sum;
};
__device__ __forceinline__ float block_max(float v, float* sh) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = -INFINITY;
  for (int i = 0; i < THREADS / 32; ++i) r = fmaxf(r, sh[i]);
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < THREADS / 32; ++i) r += sh[i];
  return r;
}
// softmax statistics of one row at temperature 1/inv_t
__device__ RowStat row_stat(const float* __restrict__ row, int V, float inv_t, float* sh) {
  float m = -INFINITY;
  for (int v = threadIdx.x; v < V; v += THREADS) m = fmaxf(m, row[v] * inv_t);
  m = block_max(m, sh);
  float s = 0.f;
  for (int v = threadIdx.x; v < V; v += THREADS) s += __expf(row[v] * inv_t - m);
  s = block_sum(s, sh);
  return {m, s};
}
// first index of the row maximum
__device__ int row_argmax(const float* __restrict__ row, int V, float* sh, int* shi) {
  float m = -INFINITY;
  int a = 0x7fffffff;
  for (int v = threadIdx.x; v < V; v += THREADS) {
    const float t = row[v];
    if (t > m) { m = t; a = v; }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const int oa = __shfl_xor_sync(0xffffffffu, a, o);
    if (om > m || (om == m && oa < a)) { m = om; a = oa; }
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { sh[threadIdx.x >> 5] = m; shi[threadIdx.x >> 5] = a; }
  __syncthreads();
  float bm = sh[0];
  int ba = shi[0];
  for (int i = 1; i < THREADS / 32; ++i)
    if (sh[i] > bm || (sh[i] == bm && shi[i] < ba)) { bm = sh[i]; ba = shi[i]; }
  return ba;
}

// Draw from the unnormalised weights f(v), v in [0,V), in index order with inverse-CDF target u * total.
// `f` is evaluated twice (total, then walk); chunks of THREADS entries are scanned in order.
template <class F>
__device__ int draw_ordered(F f, int V, float u, float* sh, int* shi) {
  float part = 0.f;
  for (int v = threadIdx.x; v < V; v += THREADS) part += f(v);
  const float total = block_sum(part, sh);
  if (!(total > 0.f)) return -1;
  const float target = u * total;
  float running = 0.f;
  int found = -1, last_pos = -1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int c0 = 0; c0 < V && found < 0; c0 += THREADS) {
    const int v = c0 + threadIdx.x;
    const float w = v < V ? f(v) : 0.f;
    // inclusive scan inside the warp, then across warps
    float incl = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) sh[warp] = incl;
    __syncthreads();
    float before = running;
    for (int i = 0; i < warp; ++i) before += sh[i];
    float chunk_total = 0.f;
    for (int i = 0; i < THREADS / 32; ++i) chunk_total += sh[i];
    const float cum = before + incl;
    const bool hit = v < V && w > 0.f && cum >= target;
    // first hitting thread of the chunk; also remember the last entry with weight for round-off fallback
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    const unsigned ballot_pos = __ballot_sync(0xffffffffu, v < V && w > 0.f);
    __syncthreads();
    if (lane == 0) {
      shi[warp] = ballot ? c0 + warp * 32 + (__ffs(ballot) - 1) : -1;
      shi[32 + warp] = ballot_pos ? c0 + warp * 32 + (31 - __clz(ballot_pos)) : -1;
    }
    __syncthreads();
    for (int i = 0; i < THREADS / 32; ++i) {
      if (found < 0 && shi[i] >= 0) found = shi[i];
      if (shi[32 + i] >= 0) last_pos = shi[32 + i];
    }
    running += chunk_total;
  }
  return found >= 0 ? found : last_pos;
}

__global__ void __launch_bounds__(THREADS)
spec_verify_kernel(const float* __restrict__ target, const float* __restrict__ draft, const int* __restrict__ tokens,
                   const float* __restrict__ uniforms, int G, int V, long ld_t, long ld_d, float inv_t, int mode,
                   int* __restrict__ n_accept, int* __restrict__ next_token) {
  __shared__ float sh[64];
  __shared__ int shi[64];
  const int b = blockIdx.x;
  const float* trow0 = target + (size_t)b * (G + 1) * ld_t;
  const float* drow0 = draft ? draft + (size_t)b * G * ld_d : nullptr;
  const int* tok = tokens + (size_t)b * G;
  const float* u = uniforms + (size_t)b * (G + 1);
  int i = 0;
  for (; i < G; ++i) {
    const float* trow = trow0 + (size_t)i * ld_t;
    int t = tok[i];
    t = t < 0 ? 0 : (t >= V ? V - 1 : t);
    if (mode == 1) {
      const int am = row_argmax(trow, V, sh, shi);
      if (am == t) continue;
      if (threadIdx.x == 0) { n_accept[b] = i; next_token[b] = am; }
      return;
    }
    const RowStat ts = row_stat(trow, V, inv_t, sh);
    const float pt = __expf(trow[t] * inv_t - ts.mx) / (ts.sum + 1e-10f);
    float pd = 1.0f / (float)V;
    RowStat ds = {0.f, 1.f};
    const float* drow = nullptr;
    if (drow0) {
      drow = drow0 + (size_t)i * ld_d;
      ds = row_stat(drow, V, inv_t, sh);
      pd = __expf(drow[t] * inv_t - ds.mx) / ds.sum;
    }
    const float accept = fminf(1.0f, pt / (pd + 1e-10f));
    if (u[i] <= accept) continue;
    // rejected: replacement from the positive part of p_target - p_draft
    const float inv_ts = 1.0f / (ts.sum + 1e-10f), inv_ds = 1.0f / ds.sum, uniform_pd = 1.0f / (float)V;
    auto residual = [&](int v) {
      const float p = __expf(trow[v] * inv_t - ts.mx) * inv_ts;
      const float q = drow ? __expf(drow[v] * inv_t - ds.mx) * inv_ds : uniform_pd;
      return fmaxf(0.f, p - q);
    };
    int r = draw_ordered(residual, V, u[G], sh, shi);
    if (r < 0) {
      auto plain = [&](int v) { return __expf(trow[v] * inv_t - ts.mx); };
      r = draw_ordered(plain, V, u[G], sh, shi);
    }
    if (threadIdx.x == 0) { n_accept[b] = i; next_token[b] = r < 0 ? t : r; }
    return;
  }
  // every draft token survived: bonus token from the target's next position
  const float* trow = trow0 + (size_t)G * ld_t;
  int r;
  if (mode == 1) {
    r = row_argmax(trow, V, sh, shi);
  } else {
    const RowStat ts = row_stat(trow, V, inv_t, sh);
    auto plain = [&](int v) { return __expf(trow[v] * inv_t - ts.mx); };
    r = draw_ordered(plain, V, u[G], sh, shi);
  }
  if (threadIdx.x == 0) { n_accept[b] = G; next_token[b] = r < 0 ? 0 : r; }
}

}  // namespace sv
}  // namespace inv

// target [B, G+1, ld_t], draft [B, G, ld_d] or null, tokens [B, G] int32, uniforms [B, G+1]; outputs int32 [B].
extern "C" int inv_spec_verify(const float* target, const float* draft, const int* tokens, const float* uniforms, int B, int G, int V, long ld_t,
                               long ld_d, float temperature, int mode, int* n_accept, int* next_token, void* stream) {
  if (B <= 0) return 0;
  if (G < 0 || V <= 0 || ld_t < V || (draft && ld_d < V) || (mode != 0 && mode != 1)) return -inv::ERR_BAD_ARG;
  const float inv_t = temperature > 0.f ? 1.0f / temperature : 1.0f;
  inv::sv::spec_verify_kernel<<<B, inv::sv::THREADS, 0, (cudaStream_t)stream>>>(target, draft, tokens, uniforms, G, V, ld_t, ld_d, inv_t, mode,
                                                                                n_accept, next_token);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
