// Gradient compression for data-parallel buckets: exact top-k sparsification and int8 quantisation.
//
// Replaces DistributedDataParallel::compress_topk_sparse / decompress_topk_sparse and compress_fp8 /
// decompress_fp8 of the reference (src/ddp.cpp:174-248): top-k keeps the k largest magnitudes of a
// bucket as (value, index) pairs and zeroes the rest in place; the int8 path stores
// round(g / (absmax / 127)) clamped to [-127, 127] with one scale per bucket.
//
// Top-k on the device is a three-level radix select on the magnitude bits (11 + 11 + 9 bits), so the
// k-th largest magnitude is found exactly with three histogram passes instead of a sort; one more
// pass compacts the survivors. All state lives in a caller-provided 4112-word scratch
// (histogram[4096] + 16 words of select state), so nothing is allocated and nothing synchronises.
// The order of the emitted pairs is not defined (the reference's is descending magnitude); the set is
// the same except among entries whose magnitude equals the k-th one.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {
namespace gc {

struct SelectState {
  uint32_t prefix;     // bits of the threshold key decided so far
  uint32_t mask;       // which bits those are
  uint32_t remaining;  // how many entries are still to be taken from the bin under refinement
  uint32_t count_out;  // pairs written so far
  uint32_t count_eq;   // entries equal to the threshold seen so far
  uint32_t k;
  uint32_t absmax_bits;
  uint32_t pad[9];
};
constexpr int HIST = 4096;

__device__ __forceinline__ uint32_t mag_key(float g) { return __float_as_uint(g) & 0x7fffffffu; }

__global__ void select_init_kernel(uint32_t* scratch, uint32_t k) {
  for (int i = threadIdx.x; i < HIST; i += blockDim.x) scratch[i] = 0;
  if (threadIdx.x == 0) {
    SelectState* s = reinterpret_cast<SelectState*>(scratch + HIST);
    s->prefix = 0; s->mask = 0; s->remaining = k; s->count_out = 0; s->count_eq = 0; s->k = k; s->absmax_bits = 0;
  }
}

__global__ void select_hist_kernel(const float* __restrict__ g, long n, uint32_t* __restrict__ scratch, int shift, int bits) {
  __shared__ uint32_t sh[2048];
  const int nb = 1 << bits;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const SelectState* s = reinterpret_cast<const SelectState*>(scratch + HIST);
  const uint32_t prefix = s->prefix, mask = s->mask;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const uint32_t key = mag_key(g[i]);
    if ((key & mask) == prefix) atomicAdd(&sh[(key >> shift) & (nb - 1)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nb; i += blockDim.x)
    if (sh[i]) atomicAdd(&scratch[i], sh[i]);
}

// One block: walk the histogram from the highest bin down to the bin that holds the remaining-th entry.
__global__ void select_pick_kernel(uint32_t* scratch, int shift, int bits) {
  __shared__ uint32_t chunk_sum[64];
  __shared__ int pick_bin;
  __shared__ uint32_t pick_above;
  SelectState* s = reinterpret_cast<SelectState*>(scratch + HIST);
  const int nb = 1 << bits;
  const int per = nb / 64;  // 64 chunks of `per` bins; thread t < 64 sums chunk t
  if (threadIdx.x < 64) {
    uint32_t c = 0;
    for (int j = 0; j < per; ++j) c += scratch[threadIdx.x * per + j];
    chunk_sum[threadIdx.x] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t want = s->remaining;
    uint32_t above = 0;
    int bin = 0;
    int c = 63;
    for (; c > 0; --c) {
      if (above + chunk_sum[c] >= want) break;
      above += chunk_sum[c];
    }
    for (bin = c * per + per - 1; bin > c * per; --bin) {
      if (above + scratch[bin] >= want) break;
      above += scratch[bin];
    }
    pick_bin = bin;
    pick_above = above;
    s->prefix |= (uint32_t)bin << shift;
    s->mask |= (uint32_t)(nb - 1) << shift;
    s->remaining = want - above;
  }
  __syncthreads();
  (void)pick_bin; (void)pick_above;
  for (int i = threadIdx.x; i < HIST; i += blockDim.x) scratch[i] = 0;
}

// Entries above the threshold are emitted; `remaining` of those equal to it are emitted; the rest are zeroed.
__global__ void select_compact_kernel(float* __restrict__ g, long n, uint32_t* __restrict__ scratch, float* __restrict__ values,
                                      int64_t* __restrict__ indices, int zero_rest) {
  SelectState* s = reinterpret_cast<SelectState*>(scratch + HIST);
  const uint32_t thr = s->prefix, take_eq = s->remaining, k = s->k;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float v = g[i];
    const uint32_t key = mag_key(v);
    bool keep = key > thr;
    if (key == thr) keep = atomicAdd(&s->count_eq, 1u) < take_eq;
    if (keep) {
      const uint32_t pos = atomicAdd(&s->count_out, 1u);
      if (pos < k) {
        values[pos] = v;
        indices[pos] = i;
      }
    } else if (zero_rest) {
      g[i] = 0.f;
    }
  }
}

__global__ void scatter_pairs_kernel(float* __restrict__ g, const float* __restrict__ values, const int64_t* __restrict__ indices, long k, long n,
                                     int accumulate) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < k; i += (long)gridDim.x * blockDim.x) {
    const int64_t j = indices[i];
    if (j >= 0 && j < n) {
      if (accumulate) atomicAdd(&g[j], values[i]);
      else g[j] = values[i];
    }
  }
}

// ---- int8 ----
__global__ void absmax_kernel(const float* __restrict__ x, long n, uint32_t* __restrict__ out_bits) {
  uint32_t m = 0;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) m = max(m, mag_key(x[i]));
#pragma unroll
  for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m) atomicMax(out_bits, m);
}
// scale_out[0] = absmax / 127 (1 when the bucket is all zero); q = clamp(round(x / scale)).
__global__ void int8_quant_kernel(const float* __restrict__ x, long n, const uint32_t* __restrict__ absmax_bits, int8_t* __restrict__ q,
                                  float* __restrict__ scale_out) {
  const float amax = __uint_as_float(*absmax_bits);
  const bool dead = amax < 1e-10f;
  const float scale = dead ? 1.0f : __fdiv_rn(amax, 127.0f);
  const float inv = __fdiv_rn(1.0f, scale);
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    int v = dead ? 0 : (int)roundf(x[i] * inv);
    v = max(-127, min(127, v));
    q[i] = (int8_t)v;
  }
}
// out[i] = sum_r q[r][i] * scale[r]  (the gathered payloads of `world` ranks, rank-major), optionally * post.
__global__ void int8_sum_dequant_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales, int world, long n, float* __restrict__ out,
                                        float post) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < world; ++r) s += (float)q[(size_t)r * n + i] * scales[r];
    out[i] = s * post;
  }
}

static inline int grid1d(long n, int block) {
  long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148L * 8 ? 148L * 8 : g));
}

}  // namespace gc
}  // namespace inv

using namespace inv::gc;

extern "C" int inv_topk_scratch_words() { return HIST + 16; }

// Keeps the k largest |g| of g[0..n): values/indices receive k pairs, g keeps only those entries when
// zero_rest is set. scratch: inv_topk_scratch_words() 32-bit words. 1 <= k <= n.
extern "C" int inv_topk_compress(float* g, long n, long k, float* values, int64_t* indices, uint32_t* scratch, int zero_rest, void* stream) {
  if (n <= 0 || k <= 0 || k > n || n >= (1L << 32)) return -inv::ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  select_init_kernel<<<1, 256, 0, st>>>(scratch, (uint32_t)k);
  const int shifts[3] = {20, 9, 0}, bits[3] = {11, 11, 9};
  const int grid = grid1d(n, 256 * 4);
  for (int p = 0; p < 3; ++p) {
    select_hist_kernel<<<grid, 256, 0, st>>>(g, n, scratch, shifts[p], bits[p]);
    select_pick_kernel<<<1, 256, 0, st>>>(scratch, shifts[p], bits[p]);
  }
  select_compact_kernel<<<grid, 256, 0, st>>>(g, n, scratch, values, indices, zero_rest);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
// g[indices[i]] = values[i] (accumulate = 0, after the caller zeroed g) or += (accumulate = 1: sum of several ranks' pairs).
extern "C" int inv_topk_scatter(float* g, long n, const float* values, const int64_t* indices, long k, int accumulate, void* stream) {
  if (k <= 0) return 0;
  scatter_pairs_kernel<<<grid1d(k, 256), 256, 0, (cudaStream_t)stream>>>(g, values, indices, k, n, accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
// scratch: one zero-initialised-by-this-call 32-bit word.
extern "C" int inv_int8_compress(const float* x, long n, int8_t* q, float* scale_out, uint32_t* scratch, void* stream) {
  if (n <= 0) return -inv::ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  cudaMemsetAsync(scratch, 0, 4, st);
  absmax_kernel<<<grid1d(n, 256 * 4), 256, 0, st>>>(x, n, scratch);
  int8_quant_kernel<<<grid1d(n, 256 * 4), 256, 0, st>>>(x, n, scratch, q, scale_out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
extern "C" int inv_int8_sum_dequant(const int8_t* q, const float* scales, int world, long n, float* out, float post, void* stream) {
  if (n <= 0 || world <= 0) return -inv::ERR_BAD_ARG;
  int8_sum_dequant_kernel<<<grid1d(n, 256 * 2), 256, 0, (cudaStream_t)stream>>>(q, scales, world, n, out, post);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
