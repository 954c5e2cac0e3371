// Batched sampler on the device: greedy argmax, temperature, top-k, top-p; repetition penalty.
//
// Replaces the reference's Sampler (src/sampler.cpp:12-122: argmax, nth_element top-k, full-sort
// top-p, repetition penalty). One CTA per row keeps the row's logits in shared memory, so that the
// selection thresholds can be found by bisection on the logit value (count >= k, mass >= p) with
// passes over shared memory instead of a sort; the token is then drawn by inverse CDF in index
// order from the kept set with a uniform number supplied by the host generator.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {

constexpr int SAMPLE_THREADS = 512;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = red[0];
  for (int w = 1; w < SAMPLE_THREADS / 32; ++w) v = is_max ? fmaxf(v, red[w]) : v + red[w];
  return v;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits, int V, int ld, float temperature, int top_k,
                                                                float top_p, const float* __restrict__ uniforms, int* __restrict__ out) {
  extern __shared__ float row[];  // V floats
  __shared__ float red[SAMPLE_THREADS / 32];
  __shared__ int red_i[SAMPLE_THREADS / 32];
  __shared__ float scan[SAMPLE_THREADS];
  const int b = blockIdx.x;
  const float* x = logits + (size_t)b * ld;
  const bool greedy = temperature <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temperature;
  float mx = -INFINITY;
  int arg = 0;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
    const float v = x[i] * inv_t;
    row[i] = v;
    if (v > mx) {
      mx = v;
      arg = i;
    }
  }
  // arg max (lowest index wins ties)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, mx, o);
    const int a2 = __shfl_xor_sync(0xffffffffu, arg, o);
    if (m2 > mx || (m2 == mx && a2 < arg)) {
      mx = m2;
      arg = a2;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    red[threadIdx.x >> 5] = mx;
    red_i[threadIdx.x >> 5] = arg;
  }
  __syncthreads();
  mx = red[0];
  arg = red_i[0];
  for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
    if (red[w] > mx || (red[w] == mx && red_i[w] < arg)) {
      mx = red[w];
      arg = red_i[w];
    }
  if (greedy) {
    if (threadIdx.x == 0) out[b] = arg;
    return;
  }
  // probabilities relative to the maximum (unnormalised): e_i = exp(row_i - mx)
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
    const float e = __expf(row[i] - mx);
    row[i] = e;
    z += e;
  }
  z = block_reduce(z, false, red);
  // Threshold on e: the kept set is {i : e_i >= thr}. Two bisections on thr in (0, 1] (the maximum has
  // e = 1): first the largest thr that still keeps top_k entries, then, within that set, the largest
  // thr whose kept mass still reaches top_p of the set's mass (top-k first, then top-p, as on the CPU).
  float thr = 0.f;
  const bool use_k = top_k > 0 && top_k < V, use_p = top_p < 1.f;
  if (use_k) {
    float lo = 0.f, hi = 1.f;
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f;
      for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) cnt += row[i] >= mid ? 1.f : 0.f;
      cnt = block_reduce(cnt, false, red);
      if (cnt >= (float)top_k) lo = mid; else hi = mid;
    }
    thr = lo;
  }
  if (use_p) {
    float zk = 0.f;
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) zk += row[i] >= thr ? row[i] : 0.f;
    zk = block_reduce(zk, false, red);
    float lo = thr, hi = 1.f;
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float mass = 0.f;
      for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) mass += row[i] >= mid ? row[i] : 0.f;
      mass = block_reduce(mass, false, red);
      if (mass >= top_p * zk) lo = mid; else hi = mid;
    }
    thr = lo;
  }
  (void)z;
  // inverse CDF over the kept entries, in index order
  float local = 0.f;
  const int per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int i0 = threadIdx.x * per, i1 = min(V, i0 + per);
  for (int i = i0; i < i1; ++i)
    if (row[i] >= thr) local += row[i];
  scan[threadIdx.x] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int t = 0; t < SAMPLE_THREADS; ++t) {
      const float v = scan[t];
      scan[t] = run;
      run += v;
    }
    red[0] = run;
    out[b] = arg;  // fallback if rounding leaves the draw outside every interval; overwritten below
  }
  __syncthreads();
  const float total = red[0];
  const float target = uniforms[b] * total;
  const float before = scan[threadIdx.x];
  if (target >= before && (target < before + local || (threadIdx.x == SAMPLE_THREADS - 1)) && local > 0.f) {
    float run = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i)
      if (row[i] >= thr) {
        pick = i;
        run += row[i];
        if (run > target) break;
      }
    if (pick >= 0) out[b] = pick;
  }
}

// logits[b, t] is divided (if positive) or multiplied (if negative) by `penalty` for every distinct
// token t in history[b, :]; a small per-row bitmap keeps repeated tokens from being penalised twice.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, int V, const int* __restrict__ history, int T, float penalty) {
  extern __shared__ uint32_t seen[];  // ceil(V/32) words
  const int b = blockIdx.x;
  const int words = (V + 31) / 32;
  for (int i = threadIdx.x; i < words; i += blockDim.x) seen[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < T; i += blockDim.x) {
    const int t = history[(size_t)b * T + i];
    if (t >= 0 && t < V) {
      const uint32_t bit = 1u << (t & 31);
      const uint32_t old = atomicOr(&seen[t >> 5], bit);
      if (!(old & bit)) {
        float* p = logits + (size_t)b * V + t;
        const float v = *p;
        *p = v > 0.f ? v / penalty : v * penalty;
      }
    }
  }
}

}  // namespace inv

using namespace inv;

extern "C" int inv_sample(const float* logits, int B, int V, int ld, float temperature, int top_k, float top_p, const float* uniforms, int* out,
                          int* status, void* stream) {
  if (B <= 0) return 0;
  const size_t smem = (size_t)V * sizeof(float);
  if (smem > 200 * 1024) return -ERR_BAD_ARG;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  sample_kernel<<<B, SAMPLE_THREADS, smem, (cudaStream_t)stream>>>(logits, V, ld, temperature, top_k, top_p, uniforms, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_repetition_penalty(float* logits, int B, int V, const int* history, int T, const int* unused, float penalty, void* stream) {
  if (B <= 0 || T <= 0) return 0;
  const size_t smem = (size_t)((V + 31) / 32) * 4;
  repetition_penalty_kernel<<<B, 256, smem, (cudaStream_t)stream>>>(logits, V, history, T, penalty);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
