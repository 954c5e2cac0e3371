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
  __syncthreads();  // x[label] has been read before anyone overwrites it
  const float inv_s = 1.f / s;
  const float g = valid ? gscale : 0.f;
  const float sm_uniform = smoothing / V;
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
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = i * 8 + j;
      float p = __expf(f[j] - m) * inv_s;
      float d = p - sm_uniform - (col == label ? (1.f - smoothing) : 0.f);
      f[j] = col < V ? d * g : 0.f;
    }
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]);
    o.y = pack_bf16x2(f[2], f[3]);
    o.z = pack_bf16x2(f[4], f[5]);
    o.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(x + i * 8) = o;
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
