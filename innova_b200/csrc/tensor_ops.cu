// General fp32 tensor operators: the arithmetic of the reference's compute-shader set as CUDA kernels.
//
// Covers the HLSL kernels of src/gpu_compute.cpp:29-176 and src/gpu_compute_full.cpp:29-348 (relu,
// gelu(tanh), silu, tanh, sigmoid, add, sub, mul, div (0 where the divisor is 0), scale, add_scalar,
// row softmax, transpose, reduce_sum / reduce_max, reduce over an axis, batch-norm over the batch
// dimension, gemv) and their CPU oracles (src/gpu_compute_vulkan.cpp:808-975). GEMM, the norms,
// embedding, attention and the MoE gather/scatter of that set live in their own files.
// Everything here is bandwidth-bound: 16-byte accesses where the shape allows, grid-stride loops,
// warp-shuffle reductions, one pass over the data except for softmax (kept in registers per row
// when it fits) and the two-stage full reductions.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {
namespace tops {

enum { U_RELU = 0, U_GELU = 1, U_SILU = 2, U_TANH = 3, U_SIGMOID = 4, U_SCALE = 5, U_ADD_SCALAR = 6, U_EXP = 7, U_SQUARE = 8 };
enum { B_ADD = 0, B_SUB = 1, B_MUL = 2, B_DIV = 3, B_MAX = 4 };
enum { R_SUM = 0, R_MAX = 1, R_MEAN = 2, R_MIN = 3 };

__device__ __forceinline__ float unary(float x, int op, float s) {
  switch (op) {
    case U_RELU: return fmaxf(x, 0.f);
    case U_GELU: return gelu_tanh(x);
    case U_SILU: return silu_f(x);
    case U_TANH: return tanhf(x);
    case U_SIGMOID: return 1.f / (1.f + __expf(-x));
    case U_SCALE: return x * s;
    case U_ADD_SCALAR: return x + s;
    case U_EXP: return __expf(x);
    default: return x * x;
  }
}
__device__ __forceinline__ float binary(float a, float b, int op) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    case B_DIV: return b != 0.f ? __fdiv_rn(a, b) : 0.f;
    default: return fmaxf(a, b);
  }
}

__global__ void unary_kernel(const float* __restrict__ x, float* __restrict__ y, long n, int op, float s) {
  const long n4 = n >> 2;
  const long tid = blockIdx.x * (long)blockDim.x + threadIdx.x, stride = (long)gridDim.x * blockDim.x;
  for (long i = tid; i < n4; i += stride) {
    float4 v = reinterpret_cast<const float4*>(x)[i];
    v.x = unary(v.x, op, s); v.y = unary(v.y, op, s); v.z = unary(v.z, op, s); v.w = unary(v.w, op, s);
    reinterpret_cast<float4*>(y)[i] = v;
  }
  for (long i = (n4 << 2) + tid; i < n; i += stride) y[i] = unary(x[i], op, s);
}
__global__ void binary_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, long n, int op) {
  const long n4 = n >> 2;
  const long tid = blockIdx.x * (long)blockDim.x + threadIdx.x, stride = (long)gridDim.x * blockDim.x;
  for (long i = tid; i < n4; i += stride) {
    const float4 u = reinterpret_cast<const float4*>(a)[i], w = reinterpret_cast<const float4*>(b)[i];
    float4 v;
    v.x = binary(u.x, w.x, op); v.y = binary(u.y, w.y, op); v.z = binary(u.z, w.z, op); v.w = binary(u.w, w.w, op);
    reinterpret_cast<float4*>(y)[i] = v;
  }
  for (long i = (n4 << 2) + tid; i < n; i += stride) y[i] = binary(a[i], b[i], op);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide combine through shared memory; result valid in every thread
__device__ __forceinline__ float block_reduce(float v, int op, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = (op == R_MAX) ? warp_max(v) : (op == R_MIN ? -warp_max(-v) : warp_sum(v));
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = (op == R_MAX) ? -INFINITY : (op == R_MIN ? INFINITY : 0.f);
  for (int i = 0; i < nw; ++i) r = (op == R_MAX) ? fmaxf(r, sh[i]) : (op == R_MIN ? fminf(r, sh[i]) : r + sh[i]);
  return r;
}

// One block per row; rows up to 8192 columns stay in registers (32 per thread), longer rows re-read.
__global__ void softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int cols) {
  __shared__ float sh[32];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* xr = x + (size_t)r * cols;
    float* yr = y + (size_t)r * cols;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, xr[c]);
    m = block_reduce(m, R_MAX, sh);
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(xr[c] - m);
    s = block_reduce(s, R_SUM, sh);
    const float inv = 1.f / s;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = __expf(xr[c] - m) * inv;
  }
}

// y[c, r] = x[r, c]; 32x32 tiles through padded shared memory, both sides coalesced.
__global__ void transpose_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int cols) {
  __shared__ float tile[32][33];
  const int tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
  for (long t = blockIdx.x; t < (long)tiles_c * tiles_r; t += gridDim.x) {
    const int r0 = (int)(t / tiles_c) * 32, c0 = (int)(t % tiles_c) * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
      const int r = r0 + j, c = c0 + threadIdx.x;
      if (r < rows && c < cols) tile[j][threadIdx.x] = x[(size_t)r * cols + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
      const int c = c0 + j, r = r0 + threadIdx.x;
      if (r < rows && c < cols) y[(size_t)c * rows + r] = tile[threadIdx.x][j];
    }
    __syncthreads();
  }
}

// Full reduction, stage 1: one partial per block. Stage 2 is the same kernel on the partials with one block.
__global__ void reduce_all_kernel(const float* __restrict__ x, float* __restrict__ out, long n, int op) {
  __shared__ float sh[32];
  float v = (op == R_MAX) ? -INFINITY : (op == R_MIN ? INFINITY : 0.f);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float t = x[i];
    v = (op == R_MAX) ? fmaxf(v, t) : (op == R_MIN ? fminf(v, t) : v + t);
  }
  v = block_reduce(v, op == R_MEAN ? R_SUM : op, sh);
  if (threadIdx.x == 0) out[blockIdx.x] = v;
}
__global__ void scale_scalar_kernel(float* v, float s) { *v *= s; }

// out[o, i] = reduce over a of x[o, a, i]. Threads run along the contiguous inner dimension when it is
// wide; for inner == 1 a warp takes one output and strides over the axis.
__global__ void reduce_axis_kernel(const float* __restrict__ x, float* __restrict__ out, long outer, int axis, long inner, int op) {
  const float init = (op == R_MAX) ? -INFINITY : (op == R_MIN ? INFINITY : 0.f);
  if (inner >= 32) {
    const long total = outer * inner;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
      const long o = i / inner, in = i % inner;
      const float* p = x + o * axis * inner + in;
      float v = init;
      for (int a = 0; a < axis; ++a) {
        const float t = p[(size_t)a * inner];
        v = (op == R_MAX) ? fmaxf(v, t) : (op == R_MIN ? fminf(v, t) : v + t);
      }
      out[i] = (op == R_MEAN) ? v / (float)axis : v;
    }
  } else {
    const int lane = threadIdx.x & 31;
    const long total = outer * inner;
    const long warp0 = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5, nwarps = ((long)gridDim.x * blockDim.x) >> 5;
    for (long i = warp0; i < total; i += nwarps) {
      const long o = i / inner, in = i % inner;
      const float* p = x + o * axis * inner + in;
      float v = init;
      for (int a = lane; a < axis; a += 32) {
        const float t = p[(size_t)a * inner];
        v = (op == R_MAX) ? fmaxf(v, t) : (op == R_MIN ? fminf(v, t) : v + t);
      }
      v = (op == R_MAX) ? warp_max(v) : (op == R_MIN ? -warp_max(-v) : warp_sum(v));
      if (lane == 0) out[i] = (op == R_MEAN) ? v / (float)axis : v;
    }
  }
}

// x[N, C, HW]: statistics over the batch dimension N for every (c, hw) position, as the reference's
// shader computes them (biased variance, eps 1e-5 by default), then affine with gamma[c], beta[c].
__global__ void batch_norm_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                  float* __restrict__ y, int N, int C, long HW, float eps) {
  const long chw = (long)C * HW;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < chw; i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i / HW);
    float s = 0.f, q = 0.f;
    for (int n = 0; n < N; ++n) {
      const float v = x[(size_t)n * chw + i];
      s += v;
      q += v * v;
    }
    const float mean = s / (float)N;
    const float var = q / (float)N - mean * mean;
    const float iv = rsqrtf(var + eps), g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
    for (int n = 0; n < N; ++n) y[(size_t)n * chw + i] = (x[(size_t)n * chw + i] - mean) * iv * g + b;
  }
}

// y[m] = sum_k A[m, k] * x[k] (+ bias[m]); one warp per row, float4 loads.
__global__ void gemv_f32_kernel(const float* __restrict__ A, const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y,
                                int M, int K) {
  const int lane = threadIdx.x & 31;
  const long warp0 = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5, nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  for (long m = warp0; m < M; m += nwarps) {
    const float* a = A + (size_t)m * K;
    float s = 0.f;
    if ((K & 3) == 0) {
      for (int k = lane * 4; k < K; k += 128) {
        const float4 u = *reinterpret_cast<const float4*>(a + k), w = *reinterpret_cast<const float4*>(x + k);
        s += u.x * w.x + u.y * w.y + u.z * w.z + u.w * w.w;
      }
    } else {
      for (int k = lane; k < K; k += 32) s += a[k] * x[k];
    }
    s = warp_sum(s);
    if (lane == 0) y[m] = s + (bias ? bias[m] : 0.f);
  }
}

static inline int grid1d(long n, int block) {
  long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148L * 16 ? 148L * 16 : g));
}

}  // namespace tops
}  // namespace inv

using namespace inv::tops;
#define RET_LAUNCH()                         \
  do {                                       \
    cudaError_t e = cudaGetLastError();      \
    return e == cudaSuccess ? 0 : -(int)e;   \
  } while (0)

extern "C" int inv_unary_f32(const float* x, float* y, long n, int op, float s, void* stream) {
  if (n <= 0) return 0;
  if (op < 0 || op > U_SQUARE || ((uintptr_t)x & 15) || ((uintptr_t)y & 15)) return -inv::ERR_BAD_ARG;
  unary_kernel<<<grid1d(n / 4 + 1, 256), 256, 0, (cudaStream_t)stream>>>(x, y, n, op, s);
  RET_LAUNCH();
}
extern "C" int inv_binary_f32(const float* a, const float* b, float* y, long n, int op, void* stream) {
  if (n <= 0) return 0;
  if (op < 0 || op > B_MAX || ((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)y & 15)) return -inv::ERR_BAD_ARG;
  binary_kernel<<<grid1d(n / 4 + 1, 256), 256, 0, (cudaStream_t)stream>>>(a, b, y, n, op);
  RET_LAUNCH();
}
extern "C" int inv_softmax_rows_f32(const float* x, float* y, int rows, int cols, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const int block = cols >= 1024 ? 256 : (cols >= 128 ? 128 : 32);
  softmax_rows_kernel<<<rows < 148 * 16 ? rows : 148 * 16, block, 0, (cudaStream_t)stream>>>(x, y, rows, cols);
  RET_LAUNCH();
}
extern "C" int inv_transpose_f32(const float* x, float* y, int rows, int cols, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const long tiles = (long)((rows + 31) / 32) * ((cols + 31) / 32);
  transpose_kernel<<<(int)(tiles < 148 * 32 ? tiles : 148 * 32), dim3(32, 8), 0, (cudaStream_t)stream>>>(x, y, rows, cols);
  RET_LAUNCH();
}
// `partials` must hold at least 1024 floats; the result lands in out[0].
extern "C" int inv_reduce_all_f32(const float* x, float* out, float* partials, long n, int op, void* stream) {
  if (n <= 0 || op < 0 || op > R_MIN) return -inv::ERR_BAD_ARG;
  int blocks = grid1d(n, 256 * 8);
  if (blocks > 1024) blocks = 1024;
  reduce_all_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, partials, n, op);
  reduce_all_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(partials, out, blocks, op);
  if (op == R_MEAN) scale_scalar_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(out, 1.0f / (float)n);
  RET_LAUNCH();
}
extern "C" int inv_reduce_axis_f32(const float* x, float* out, long outer, int axis, long inner, int op, void* stream) {
  if (outer <= 0 || axis <= 0 || inner <= 0 || op < 0 || op > R_MIN) return -inv::ERR_BAD_ARG;
  const long work = inner >= 32 ? outer * inner : outer * inner * 32;
  reduce_axis_kernel<<<grid1d(work, 256), 256, 0, (cudaStream_t)stream>>>(x, out, outer, axis, inner, op);
  RET_LAUNCH();
}
extern "C" int inv_batch_norm_f32(const float* x, const float* gamma, const float* beta, float* y, int N, int C, long HW, float eps,
                                  void* stream) {
  if (N <= 0 || C <= 0 || HW <= 0) return -inv::ERR_BAD_ARG;
  batch_norm_kernel<<<grid1d((long)C * HW, 256), 256, 0, (cudaStream_t)stream>>>(x, gamma, beta, y, N, C, HW, eps);
  RET_LAUNCH();
}
extern "C" int inv_gemv_f32(const float* A, const float* x, const float* bias, float* y, int M, int K, void* stream) {
  if (M <= 0 || K <= 0) return -inv::ERR_BAD_ARG;
  if ((K & 3) == 0 && (((uintptr_t)A & 15) || ((uintptr_t)x & 15))) return -inv::ERR_BAD_ARG;
  gemv_f32_kernel<<<grid1d((long)M * 32, 256), 256, 0, (cudaStream_t)stream>>>(A, x, bias, y, M, K);
  RET_LAUNCH();
}
