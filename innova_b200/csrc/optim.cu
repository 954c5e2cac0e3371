// Fused optimizer kernels over flat fp32 buffers: gradient sum of squares (for the global-norm
// clip) and an AdamW step that reads the fp32 gradient, updates fp32 master weights and moments,
// writes the bf16 compute copy and clears the gradient, all in one pass.
//
// Replaces the reference's AdamW::step (src/optimizer.cpp:91-119) and the base-class global-norm
// clip (src/optimizer.cpp:20-42). Hyper-parameters are read from device memory so that a captured
// CUDA graph can be replayed while the host changes the learning rate between steps.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {

// hyper layout (floats): 0 lr_adj (lr / bias_corr1, times sqrt(bias_corr2) in reference mode),
// 1 beta1, 2 beta2, 3 eps, 4 lr*weight_decay, 5 1/bias_corr2, 6 max_norm (<=0: no clip),
// 7 grad_scale (e.g. 1/loss_scale or 1/world), 8 decay_after (1: p -= lr*wd*p after the update,
// as the reference does; 0: decoupled decay before the update).
__global__ void sumsq_kernel(const float* __restrict__ g, long n, float* __restrict__ out) {
  float s = 0.f;
  const long n4 = n / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 v = reinterpret_cast<const float4*>(g)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long i = n4 * 4; i < n; ++i) s += g[i] * g[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

__device__ __forceinline__ float adamw_one(float& p, float& m, float& v, float g, float lr_adj, float b1, float b2, float eps, float lrwd,
                                           float inv_bc2, bool decay_after) {
  if (!decay_after) p -= lrwd * p;
  m = b1 * m + (1.f - b1) * g;
  v = b2 * v + (1.f - b2) * g * g;
  p -= lr_adj * m / (sqrtf(v * inv_bc2) + eps);
  if (decay_after) p -= lrwd * p;
  return p;
}

__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, float* __restrict__ g,
                             __nv_bfloat16* __restrict__ p16, long n, const float* __restrict__ hyper, const float* __restrict__ gnorm_sq,
                             int zero_grad) {
  const float lr_adj = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], lrwd = hyper[4], inv_bc2 = hyper[5];
  const float max_norm = hyper[6];
  float gs = hyper[7];
  const bool decay_after = hyper[8] != 0.f;
  if (max_norm > 0.f && gnorm_sq != nullptr) {
    const float norm = sqrtf(*gnorm_sq) * gs;
    gs *= fminf(1.f, max_norm / (norm + 1e-6f));
  }
  const long n4 = n / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i], mv = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
    float4 gv = reinterpret_cast<float4*>(g)[i];
    adamw_one(pv.x, mv.x, vv.x, gv.x * gs, lr_adj, b1, b2, eps, lrwd, inv_bc2, decay_after);
    adamw_one(pv.y, mv.y, vv.y, gv.y * gs, lr_adj, b1, b2, eps, lrwd, inv_bc2, decay_after);
    adamw_one(pv.z, mv.z, vv.z, gv.z * gs, lr_adj, b1, b2, eps, lrwd, inv_bc2, decay_after);
    adamw_one(pv.w, mv.w, vv.w, gv.w * gs, lr_adj, b1, b2, eps, lrwd, inv_bc2, decay_after);
    reinterpret_cast<float4*>(p)[i] = pv;
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p16) {
      uint2 o;
      o.x = pack_bf16x2(pv.x, pv.y);
      o.y = pack_bf16x2(pv.z, pv.w);
      reinterpret_cast<uint2*>(p16)[i] = o;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long i = n4 * 4; i < n; ++i) {
      float pv = p[i], mv = m[i], vv = v[i];
      adamw_one(pv, mv, vv, g[i] * gs, lr_adj, b1, b2, eps, lrwd, inv_bc2, decay_after);
      p[i] = pv; m[i] = mv; v[i] = vv;
      if (zero_grad) g[i] = 0.f;
      if (p16) p16[i] = __float2bfloat16_rn(pv);
    }
  }
}

}  // namespace inv

using namespace inv;

extern "C" int inv_sumsq(const float* g, long n, float* out, void* stream) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(g) & 15) return -ERR_BAD_ARG;
  sumsq_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>(g, n, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_adamw(float* p, float* m, float* v, float* g, void* p16, long n, const float* hyper, const float* gnorm_sq, int zero_grad,
                         void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(g)) & 15)
    return -ERR_BAD_ARG;
  if (p16 && (reinterpret_cast<uintptr_t>(p16) & 7)) return -ERR_BAD_ARG;
  adamw_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(p, m, v, g, (__nv_bfloat16*)p16, n, hyper, gnorm_sq, zero_grad);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
