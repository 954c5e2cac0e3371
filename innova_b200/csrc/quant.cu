// Train-in-format quantisation kernels: block-wise codebook quantise / dequantise and the
// straight-through fake-quant forward.
//
// Compute format (the reference's in-memory engines, src/oil_engines_oil8.cpp:42-140,
// src/oil_engines_core.cpp:15-160, used by STEQuantizer, src/ste_quantizer.cpp:19-66,145-202):
// weights are cut into blocks of 32 consecutive values; a block stores its abs-max as scale, and every
// value stores the index of the nearest entry of a shared codebook over the normalised range [-1, 1]
// (256 entries for OIL8, 16 for OIL4). SPARK is ternary {-s, 0, +s} with a 0.5*max dead zone, OIL1 is
// sign times the block's mean magnitude.
//
// One warp owns one block (lane = element): abs-max by shuffles, nearest entry by binary search over
// the sorted codebook held in shared memory. Modes: 0 OIL8, 1 OIL4, 2 SPARK, 3 OIL1.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Index of the codebook entry nearest to x; cb is sorted ascending, K is a power of two.
__device__ __forceinline__ int nearest_sorted(const float* cb, int K, float x) {
  int lo = 0;
  for (int step = K >> 1; step > 0; step >>= 1)
    if (cb[lo + step] <= x) lo += step;
  if (lo + 1 < K && (cb[lo + 1] - x) < (x - cb[lo])) ++lo;
  return lo;
}

// in: fp32 or bf16 weights (n values). out_q (bf16 or fp32, optional): dequantised values.
// idx (optional): one byte per value. scales (optional): one float per block of 32.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) block_quant_kernel(const TIn* __restrict__ in, TOut* __restrict__ out_q, uint8_t* __restrict__ idx,
                                                          float* __restrict__ scales, const float* __restrict__ codebook, int K, long n,
                                                          int mode) {
  __shared__ float cb[256];
  for (int i = threadIdx.x; i < K; i += blockDim.x) cb[i] = codebook ? codebook[i] : 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long nblocks = (n + 31) / 32;
  for (long b = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5); b < nblocks; b += (long)gridDim.x * (blockDim.x >> 5)) {
    const long i = b * 32 + lane;
    const bool ok = i < n;
    const float w = ok ? (float)in[i] : 0.f;
    const float amax = warp_max(fabsf(w));
    const bool dead = amax < 1e-10f;  // an all-zero block keeps scale 0, so that it dequantises to exactly zero
    float scale = dead ? 1.f : amax;
    float q;
    int code;
    if (mode <= 1) {
      code = nearest_sorted(cb, K, w / scale);
      if (dead) scale = 0.f;
      q = cb[code] * scale;
    } else if (mode == 2) {
      const bool keep = fabsf(w) > 0.5f * amax && amax > 0.f;
      const float cnt = warp_add(keep ? 1.f : 0.f);
      const float mag = warp_add(keep ? fabsf(w) : 0.f);
      scale = cnt > 0.f ? mag / cnt : 0.f;
      code = keep ? (w > 0.f ? 1 : 2) : 0;
      q = keep ? copysignf(scale, w) : 0.f;
    } else {
      const int cntn = (int)min(32L, n - b * 32);
      scale = warp_add(fabsf(w)) / (float)cntn;
      code = w >= 0.f ? 1 : 0;
      q = w >= 0.f ? scale : -scale;
    }
    if (ok) {
      if (out_q) out_q[i] = (TOut)q;
      if (idx) idx[i] = (uint8_t)code;
    }
    if (scales && lane == 0) scales[b] = scale;
  }
}

// out[i] = codebook[idx[i]] * scales[i / 32]   (OIL8 / OIL4 compute format -> bf16)
__global__ void block_dequant_kernel(const uint8_t* __restrict__ idx, const float* __restrict__ scales, const float* __restrict__ codebook, int K,
                                     __nv_bfloat16* __restrict__ out, long n) {
  __shared__ float cb[256];
  for (int i = threadIdx.x; i < K; i += blockDim.x) cb[i] = codebook[i];
  __syncthreads();
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(cb[idx[i] & (K - 1)] * scales[i >> 5]);
}

// Packs one-byte OIL4 indices into nibbles: out[i] = idx[2i] | idx[2i+1] << 4.
__global__ void pack_nibbles_kernel(const uint8_t* __restrict__ idx, uint8_t* __restrict__ out, long n2) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n2; i += (long)gridDim.x * blockDim.x)
    out[i] = (uint8_t)((idx[2 * i] & 15) | (idx[2 * i + 1] << 4));
}

}  // namespace inv

using namespace inv;

// in_dtype / out_dtype: 0 = fp32, 1 = bf16. Any of out_q, idx, scales may be null.
extern "C" int inv_block_quant(const void* in, int in_dtype, void* out_q, int out_dtype, uint8_t* idx, float* scales, const float* codebook,
                               int K, long n, int mode, void* stream) {
  if (n <= 0) return 0;
  if (mode < 0 || mode > 3 || (mode <= 1 && (codebook == nullptr || (K != 16 && K != 256)))) return -ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  long blocks = ((n + 31) / 32 + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const int g = (int)blocks;
  if (in_dtype == 0 && out_dtype == 0)
    block_quant_kernel<float, float><<<g, 256, 0, st>>>((const float*)in, (float*)out_q, idx, scales, codebook, K, n, mode);
  else if (in_dtype == 0 && out_dtype == 1)
    block_quant_kernel<float, __nv_bfloat16><<<g, 256, 0, st>>>((const float*)in, (__nv_bfloat16*)out_q, idx, scales, codebook, K, n, mode);
  else if (in_dtype == 1 && out_dtype == 1)
    block_quant_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out_q, idx, scales, codebook,
                                                                       K, n, mode);
  else
    block_quant_kernel<__nv_bfloat16, float><<<g, 256, 0, st>>>((const __nv_bfloat16*)in, (float*)out_q, idx, scales, codebook, K, n, mode);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_block_dequant(const uint8_t* idx, const float* scales, const float* codebook, int K, void* out, long n, void* stream) {
  if (n <= 0) return 0;
  if (K != 16 && K != 256) return -ERR_BAD_ARG;
  long g = (n + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  block_dequant_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>(idx, scales, codebook, K, (__nv_bfloat16*)out, n);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_pack_nibbles(const uint8_t* idx, uint8_t* out, long n, void* stream) {
  if (n <= 0) return 0;
  if (n & 1) return -ERR_BAD_ARG;
  long g = (n / 2 + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  pack_nibbles_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>(idx, out, n / 2);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
