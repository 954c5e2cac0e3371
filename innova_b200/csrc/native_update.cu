// Train-in-format weight store on the device: weights exist only as (format, scale, index) per block,
// and the optimizer step is the reference's two-timescale update.
//
// Replaces NativeOILWeightStore::convert_from_fp32 / dequantize / apply_oil_update
// (src/native_weight.cpp:237-272,274-285,287-335) and dead_zone_radius (include/oil/native_weight.h:50-57).
// Per block of `block_size` weights: format in {0: OIL1 ternary {-1,0,+1}, 1: OIL4 16-entry codebook,
// 2: OIL8 256-entry codebook}, one fp32 abs-max scale, one index byte per weight.
//
// Update of one block, element i in storage order (this is what the reference's loop does, including
// the fact that the shared scale moves while the loop walks the block):
//     s_before_i = scale after elements < i          w_i = s_before_i * cb[idx_i]
//     scale     -= lr_scale * g_i * cb[idx_i] / block_size      (floor 1e-10)
//     if |lr_weight * g_i| > dead_zone(fmt, s_before_i):  idx_i = nearest(cb, (w_i - lr_weight*g_i) / scale_after_i)
// One warp owns one block. Each lane takes a contiguous run of elements and the running scale is
// rebuilt from a warp prefix sum of g*cb, so the result equals the sequential loop up to fp32
// summation order (and to where the 1e-10 floor would bind mid-block, which needs a scale that small).
// nearest() returns the first entry at minimal distance like the reference's linear scan; codebooks
// must be ascending (the uniform, quantile and k-means codebooks all are), which lets OIL8 use a
// binary search plus a neighbour check instead of 256 compares.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {
namespace nw {

__device__ __forceinline__ int nearest_sorted(const float* cb, int K, float v) {
  // first index with cb[idx] >= v
  int lo = 0, hi = K;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (cb[mid] < v) lo = mid + 1; else hi = mid;
  }
  if (lo == 0) return 0;
  if (lo == K) {  // above the top entry: walk down over equal entries to the first of them
    int b = K - 1;
    while (b > 0 && cb[b - 1] == cb[b]) --b;
    return b;
  }
  const float dl = fabsf(v - cb[lo - 1]), dh = fabsf(v - cb[lo]);
  int b = (dh < dl) ? lo : lo - 1;  // tie -> lower index, as a forward linear scan with strict '<' gives
  while (b > 0 && cb[b - 1] == cb[b]) --b;
  return b;
}
__device__ __forceinline__ int quantise(int fmt, const float* cb4, const float* cb8, float norm) {
  if (fmt == 0) return norm > 0.5f ? 2 : (norm < -0.5f ? 0 : 1);
  return fmt == 1 ? nearest_sorted(cb4, 16, norm) : nearest_sorted(cb8, 256, norm);
}
__device__ __forceinline__ float centroid(int fmt, const float* cb4, const float* cb8, int idx) {
  if (fmt == 0) return (float)idx - 1.0f;
  return fmt == 1 ? cb4[idx & 15] : cb8[idx & 255];
}
__device__ __forceinline__ float dead_zone(int fmt, float s) { return s * (fmt == 2 ? 0.00390625f : (fmt == 0 ? 0.5f : 0.0625f)); }

struct Codebooks {
  float cb4[16];
  float cb8[256];
};
__device__ __forceinline__ void load_codebooks(Codebooks* sh, const float* cb4, const float* cb8) {
  for (int i = threadIdx.x; i < 16; i += blockDim.x) sh->cb4[i] = cb4[i];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) sh->cb8[i] = cb8[i];
  __syncthreads();
}

// scale = abs-max of the block (1 when < 1e-10); idx = quantise(w / scale).
__global__ void native_convert_kernel(const float* __restrict__ w, long n, int bs, const uint8_t* __restrict__ fmt, const float* __restrict__ cb4,
                                      const float* __restrict__ cb8, float* __restrict__ scales, uint8_t* __restrict__ idx) {
  __shared__ Codebooks cbs;
  load_codebooks(&cbs, cb4, cb8);
  const int lane = threadIdx.x & 31;
  const long nblocks = (n + bs - 1) / bs;
  const long warp0 = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5, nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  for (long b = warp0; b < nblocks; b += nwarps) {
    const long base = b * bs;
    const int cnt = (int)min((long)bs, n - base);
    float m = 0.f;
    for (int i = lane; i < cnt; i += 32) m = fmaxf(m, fabsf(w[base + i]));
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float s = m > 1e-10f ? m : 1.0f;
    if (lane == 0) scales[b] = s;
    const int f = fmt[b];
    for (int i = lane; i < cnt; i += 32) idx[base + i] = (uint8_t)quantise(f, cbs.cb4, cbs.cb8, __fdiv_rn(w[base + i], s));
  }
}

// out = scale * centroid; out_bf16 selects the element type of `out`.
__global__ void native_dequant_kernel(const uint8_t* __restrict__ idx, const float* __restrict__ scales, const uint8_t* __restrict__ fmt, long n,
                                      int bs, const float* __restrict__ cb4, const float* __restrict__ cb8, void* __restrict__ out, int out_bf16) {
  __shared__ Codebooks cbs;
  load_codebooks(&cbs, cb4, cb8);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long b = i / bs;
    const float v = scales[b] * centroid(fmt[b], cbs.cb4, cbs.cb8, idx[i]);
    if (out_bf16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(out)[i] = v;
  }
}

__global__ void native_update_kernel(const float* __restrict__ grad, long n, int bs, const uint8_t* __restrict__ fmt, const float* __restrict__ cb4,
                                     const float* __restrict__ cb8, float* __restrict__ scales, uint8_t* __restrict__ idx,
                                     const uint8_t* __restrict__ frozen, float lr_scale, float lr_weight, unsigned long long* __restrict__ changed) {
  __shared__ Codebooks cbs;
  load_codebooks(&cbs, cb4, cb8);
  const int lane = threadIdx.x & 31;
  const long nblocks = (n + bs - 1) / bs;
  const long warp0 = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5, nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  const int per = (bs + 31) / 32;  // contiguous elements per lane
  unsigned int flips = 0;
  for (long b = warp0; b < nblocks; b += nwarps) {
    const long base = b * bs;
    const int cnt = (int)min((long)bs, n - base);
    const int f = fmt[b];
    const float s0 = scales[b];
    const float step = lr_scale / (float)bs;
    const int i0 = lane * per, i1 = min(cnt, i0 + per);
    // lane-local sum of g*cv, then exclusive prefix over lanes
    float local = 0.f;
    for (int i = i0; i < i1; ++i) local += grad[base + i] * centroid(f, cbs.cb4, cbs.cb8, idx[base + i]);
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    float run = incl - local;  // sum over all elements before this lane's run
    for (int i = i0; i < i1; ++i) {
      const int id = idx[base + i];
      const float cv = centroid(f, cbs.cb4, cbs.cb8, id);
      const float g = grad[base + i];
      const float s_before = fmaxf(s0 - step * run, 1e-10f);
      run += g * cv;
      const float s_after = fmaxf(s0 - step * run, 1e-10f);
      if (frozen == nullptr || !frozen[base + i]) {
        const float w = s_before * cv;
        const float wv = w - lr_weight * g;
        if (fabsf(wv - w) > dead_zone(f, s_before)) {
          const int ni = quantise(f, cbs.cb4, cbs.cb8, __fdiv_rn(wv, s_after));
          if (ni != id) {
            idx[base + i] = (uint8_t)ni;
            ++flips;
          }
        }
      }
    }
    const float total = __shfl_sync(0xffffffffu, incl, 31);
    if (lane == 0) scales[b] = fmaxf(s0 - step * total, 1e-10f);
  }
  if (changed) {
#pragma unroll
    for (int o = 16; o; o >>= 1) flips += __shfl_xor_sync(0xffffffffu, flips, o);
    if (lane == 0 && flips) atomicAdd(changed, (unsigned long long)flips);
  }
}

static inline int grid1d(long n, int block) {
  long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148L * 8 ? 148L * 8 : g));
}
}  // namespace nw
}  // namespace inv

using namespace inv::nw;

extern "C" int inv_native_convert(const float* w, long n, int block_size, const uint8_t* fmt, const float* cb4, const float* cb8, float* scales,
                                  uint8_t* idx, void* stream) {
  if (n <= 0 || block_size < 1) return -inv::ERR_BAD_ARG;
  const long nblocks = (n + block_size - 1) / block_size;
  native_convert_kernel<<<grid1d(nblocks * 32, 256), 256, 0, (cudaStream_t)stream>>>(w, n, block_size, fmt, cb4, cb8, scales, idx);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
extern "C" int inv_native_dequant(const uint8_t* idx, const float* scales, const uint8_t* fmt, long n, int block_size, const float* cb4,
                                  const float* cb8, void* out, int out_bf16, void* stream) {
  if (n <= 0 || block_size < 1) return -inv::ERR_BAD_ARG;
  native_dequant_kernel<<<grid1d(n, 256 * 4), 256, 0, (cudaStream_t)stream>>>(idx, scales, fmt, n, block_size, cb4, cb8, out, out_bf16);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
// changed (optional): device counter that receives the number of indices that moved.
extern "C" int inv_native_update(const float* grad, long n, int block_size, const uint8_t* fmt, const float* cb4, const float* cb8, float* scales,
                                 uint8_t* idx, const uint8_t* frozen, float lr_scale, float lr_weight, unsigned long long* changed, void* stream) {
  if (n <= 0 || block_size < 1) return -inv::ERR_BAD_ARG;
  const long nblocks = (n + block_size - 1) / block_size;
  native_update_kernel<<<grid1d(nblocks * 32, 256), 256, 0, (cudaStream_t)stream>>>(grad, n, block_size, fmt, cb4, cb8, scales, idx, frozen,
                                                                                     lr_scale, lr_weight, changed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
