// Fused softmax cross-entropy over bf16 logits: one pass for the statistics, one pass that
// overwrites the logits with their gradient. Nothing of size [T, V] is allocated.
//
// Replaces the reference's cross_entropy_loss / cross_entropy_grad (src/autograd_grad.cpp:220-271:
// mean over positions of logsumexp - logit[target], grad = (softmax - onehot) / count) and the
// vk_cross_entropy pair (src/gpu_compute_vulkan.cpp:1156-1202). Label smoothing follows the
// reference trainer's option (src/trainer_core.cpp:408-474).
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {

constexpr int CE_THREADS = 512;

// logits: [T, ld] bf16, columns [V, ld) are padding. labels < 0 are ignored.
// loss[t] = (1-eps)*nll + eps*(lse - mean(x));  if grad != 0: logits <- dloss/dlogits * gscale.
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ labels,
                                                                   float* __restrict__ loss, float* __restrict__ lse_out, int V, int ld,
                                                                   float gscale, float smoothing, int write_grad) {
  __shared__ float sm_m[CE_THREADS / 32], sm_s[CE_THREADS / 32], sm_x[CE_THREADS / 32];
  __shared__ float bc[3];
  const int row = blockIdx.x;
  __nv_bfloat16* x = logits + (size_t)row * ld;
  const long label = labels[row];
  const int nvec = ld / 8;
  float m = -INFINITY, s = 0.f, sx = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    uint4 v = *reinterpret_cast<const uint4*>(x + i * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
    float lm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i * 8 + j < V) lm = fmaxf(lm, f[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i * 8 + j < V) {
        s += __expf(f[j] - m);
        sx += f[j];
      }
  }
  // warp then block reduction of (m, s) pairs
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    sx += __shfl_xor_sync(0xffffffffu, sx, o);
    float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
    m = mn;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sm_m[warp] = m;
    sm_s[warp] = s;
    sm_x[warp] = sx;
  }
  __syncthreads();
  if (warp == 0) {
    m = lane < CE_THREADS / 32 ? sm_m[lane] : -INFINITY;
    s = lane < CE_THREADS / 32 ? sm_s[lane] : 0.f;
    sx = lane < CE_THREADS / 32 ? sm_x[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      sx += __shfl_xor_sync(0xffffffffu, sx, o);
      float mn = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
      m = mn;
    }
    if (lane == 0) {
      bc[0] = m;
      bc[1] = s;
      bc[2] = sx;
    }
  }
  __syncthreads();
  m = bc[0];
  s = bc[1];
  sx = bc[2];
  const float lse = m + __logf(s);
  const bool valid = label >= 0 && label < V;
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (valid) {
      const float xl = __bfloat162float(x[label]);
      l = (1.f - smoothing) * (lse - xl) + smoothing * (lse - sx / V);
    }
    loss[row] = l;
    if (lse_out) lse_out[row] = lse;
  }
  if (!write_grad) return;
  // Second pass: p = exp2(x * log2(e) - (m * log2(e) + log2(s))) with the packed bf16x2 exponential: two results per
  // MUFU instruction, and the result is stored as bf16 anyway. (With one fp32 exponential per element in each pass the
  // kernel was bound by the special-function unit, not by memory.) The label's column is rewritten in fp32 afterwards.
  const float g = valid ? gscale : 0.f;
  const float kL2E = 1.4426950408889634f;
  const float c = -(m * kL2E + __log2f(s));
  const uint32_t g2 = pack_bf16x2(g, g);
  const uint32_t ug2 = pack_bf16x2(-g * smoothing / V, -g * smoothing / V);
  const float xl = valid ? __bfloat162float(x[label]) : 0.f;
  __syncthreads();  // x[label] has been read by every thread before anyone overwrites it
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    uint4 v = *reinterpret_cast<const uint4*>(x + i * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(h[j]);
      const uint32_t e = ex2_bf16x2(pack_bf16x2_int(fmaf(t.x, kL2E, c), fmaf(t.y, kL2E, c)));
      asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o[j]) : "r"(e), "r"(g2), "r"(ug2));
    }
    if (i * 8 + 8 > V) {  // the vector that straddles the end of the vocabulary, and the padding behind it
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (i * 8 + 2 * j >= V) o[j] = 0u;
        else if (i * 8 + 2 * j + 1 >= V) o[j] &= 0x0000ffffu;
      }
    }
    *reinterpret_cast<uint4*>(x + i * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (valid) {
    __syncthreads();
    if (threadIdx.x == 0) {
      const float pl = __expf(xl - m) / s;
      x[label] = __float2bfloat16((pl - smoothing / V - (1.f - smoothing)) * g);
    }
  }
}

}  // namespace inv

using namespace inv;

extern "C" int inv_cross_entropy(void* logits, const int64_t* labels, float* loss, float* lse, int T, int V, int ld, float gscale,
                                 float smoothing, int write_grad, void* stream) {
  if (ld % 8 || V > ld) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  cross_entropy_kernel<<<T, CE_THREADS, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, labels, loss, lse, V, ld, gscale, smoothing,
                                                                   write_grad);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
