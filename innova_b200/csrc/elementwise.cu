// Memory-bound operators around the GEMMs: embedding gather / scatter-add, bias-gradient column
// sums, GELU / SwiGLU forward and backward, half-split RoPE, and small utilities.
//
// Replaces the reference's Embedding (src/transformer.cpp:32-49), simd::swiglu / silu_grad /
// gelu_grad (src/simd_math.cpp:146-186, src/autograd_grad.cpp:89-117), RotaryEmbedding::apply and
// RotaryFunction (src/transformer.cpp:129-171, src/autograd_functions.cpp:360-396), and the shader
// parity set embedding / transpose / reduce (src/gpu_compute_full.cpp:120-263).
// All kernels use 16-byte accesses (8 bf16) and grid-stride loops.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float* f) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float* f) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// out[t,:] = wte[ids[t],:] (+ wpe[t % S,:]). Ids outside [0,V) read row 0, as the reference does.
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, int T, int S, int D, int V) {
  const int vec_per_row = D / 8;
  const long total = (long)T * vec_per_row;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec_per_row);
    const int c = (int)(i % vec_per_row) * 8;
    long id = ids[t];
    if (id < 0 || id >= V) id = 0;
    float a[8];
    ld8(wte + id * D + c, a);
    if (wpe) {
      float b[8];
      ld8(wpe + (size_t)(t % S) * D + c, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
    }
    st8(out + (size_t)t * D + c, a);
  }
}

// dwte[ids[t],:] += dy[t,:] (vector reductions); dwpe[s,:] += sum_b dy[b*S+s,:].
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ dy, float* __restrict__ dwte,
                                     float* __restrict__ dwpe, int T, int S, int D, int V) {
  const int vec_per_row = D / 8;
  const int nb = T / S;
  const long total = (long)S * vec_per_row;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int s = (int)(i / vec_per_row);
    const int c = (int)(i % vec_per_row) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = 0; b < nb; ++b) {
      const int t = b * S + s;
      float a[8];
      ld8(dy + (size_t)t * D + c, a);
      long id = ids[t];
      if (id < 0 || id >= V) id = 0;
      float* dst = dwte + id * D + c;
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a[0]), "f"(a[1]), "f"(a[2]), "f"(a[3]) : "memory");
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(a[4]), "f"(a[5]), "f"(a[6]), "f"(a[7]) : "memory");
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += a[j];
    }
    if (dwpe) {
      float* dst = dwpe + (size_t)s * D + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] += acc[j];
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}

// out[n] += sum_t x[t,n]   (bias gradient). grid = (ceil(N/256), row_chunks), block = 256: a lane owns 8 columns (one 16-byte
// load per row), a warp 256 columns, the 8 warps of a CTA take rows round robin with four rows in flight each; the CTA's
// 256 partial sums meet in shared memory and leave as one atomic per column.
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int T, int N, int ld,
                                                      int rows_per_block) {
  __shared__ float red[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(T, r0 + rows_per_block);
  float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < N) {  // N % 8 == 0: a lane's 8 columns are inside or outside together
    const __nv_bfloat16* base = x + col;
    int r = r0 + warp;
    for (; r + 24 < r1; r += 32) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(base + (size_t)(r + 8 * u) * ld);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8];
        unpack8(v[u], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] += f[j];
      }
    }
    for (; r < r1; r += 8) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(base + (size_t)r * ld), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += f[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = a[j];
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) atomicAdd(out + c, s);
}

// The same for rows that are not 16-byte friendly (N or ld not a multiple of 8): two columns per lane.
__global__ void __launch_bounds__(256) colsum2_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int T, int N, int ld,
                                                       int rows_per_block) {
  __shared__ float red[8][64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + lane * 2;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(T, r0 + rows_per_block);
  float a0 = 0.f, a1 = 0.f;
  if (col < N) {
    for (int r = r0 + warp; r < r1; r += 8) {
      float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (size_t)r * ld + col));
      a0 += f.x;
      a1 += f.y;
    }
  }
  red[warp][lane * 2] = a0;
  red[warp][lane * 2 + 1] = a1;
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < N) atomicAdd(out + c, s);
  }
}

// mode 0: y = gelu(x); 1: dx = dy * gelu'(x); 2: y = silu(g) * u (x = [g | u] halves of a 2F row);
// 3: SwiGLU backward: d[g|u] from dy, g, u.
// rows_dev != nullptr: only the first min(rows, *rows_dev) rows are processed (a row count that lives on the device).
__global__ void act_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ out, long rows,
                           int F, int mode, const int* __restrict__ rows_dev) {
  const int vec = F / 8;
  if (rows_dev != nullptr) rows = min(rows, (long)*rows_dev);
  const long total = rows * vec;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / vec;
    const int c = (int)(i % vec) * 8;
    if (mode == 0 || mode == 1) {
      float a[8], o[8];
      ld8(x + r * F + c, a);
      if (mode == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = gelu_tanh(a[j]);
      } else {
        float d[8];
        ld8(dy + r * F + c, d);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = d[j] * gelu_tanh_grad(a[j]);
      }
      st8(out + r * F + c, o);
    } else {
      float g[8], u[8];
      ld8(x + r * 2 * F + c, g);
      ld8(x + r * 2 * F + F + c, u);
      if (mode == 2) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = silu_f(g[j]) * u[j];
        st8(out + r * F + c, o);
      } else {
        float d[8], dg[8], du[8];
        ld8(dy + r * F + c, d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dg[j] = d[j] * u[j] * silu_grad_f(g[j]);
          du[j] = d[j] * silu_f(g[j]);
        }
        st8(out + r * 2 * F + c, dg);
        st8(out + r * 2 * F + F + c, du);
      }
    }
  }
}

// Half-split rotary embedding applied in place to `nheads` heads starting at column `col0` of a
// token-major buffer [T, ld]: (x1, x2) -> (x1 c - x2 s, x1 s + x2 c), x1 = first half of the head.
// pos[t] gives the position (or t % S when pos is null). inverse = 1 applies the transpose (backward).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ pos, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, int T, int S, int ld, int col0, int nheads, int hd, int inverse) {
  const int half = hd / 2;
  const int vec_per_head = half / 8;
  const long total = (long)T * nheads * vec_per_head;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const long r = i / vec_per_head;
    const int h = (int)(r % nheads);
    const int t = (int)(r / nheads);
    const int p = pos ? pos[t] : (t % S);
    __nv_bfloat16* base = buf + (size_t)t * ld + col0 + h * hd + v * 8;
    float x1[8], x2[8], o1[8], o2[8];
    ld8(base, x1);
    ld8(base + half, x2);
    const float* cp = cos_t + (size_t)p * half + v * 8;
    const float* sp = sin_t + (size_t)p * half + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = cp[j];
      const float s = inverse ? -sp[j] : sp[j];
      o1[j] = x1[j] * c - x2[j] * s;
      o2[j] = x1[j] * s + x2[j] * c;
    }
    st8(base, o1);
    st8(base + half, o2);
  }
}

// y = a + b (bf16), used where a residual add cannot ride in a GEMM epilogue.
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, long n8) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float x[8], z[8];
    ld8(a + i * 8, x);
    ld8(b + i * 8, z);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += z[j];
    st8(y + i * 8, x);
  }
}

// Writes `bytes` of a scratch buffer; used to evict L2 between timed iterations.
__global__ void l2_flush_kernel(uint4* buf, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) buf[i] = make_uint4(i, 0, 0, 0);
}

static inline int grid_for(long n, int block) {
  long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148L * 16 ? 148L * 16 : g));
}

}  // namespace inv

using namespace inv;
#define CHECK_LAUNCH()                       \
  do {                                       \
    cudaError_t e = cudaGetLastError();      \
    return e == cudaSuccess ? 0 : -(int)e;   \
  } while (0)

extern "C" int inv_embedding_fwd(const int64_t* ids, const void* wte, const void* wpe, void* out, int T, int S, int D, int V, void* stream) {
  if (D % 8) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<grid_for((long)T * D / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      ids, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out, T, S, D, V);
  CHECK_LAUNCH();
}
extern "C" int inv_embedding_bwd(const int64_t* ids, const void* dy, float* dwte, float* dwpe, int T, int S, int D, int V, void* stream) {
  if (D % 8 || S <= 0 || T % S) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  embedding_bwd_kernel<<<grid_for((long)S * D / 8, 128), 128, 0, (cudaStream_t)stream>>>(ids, (const __nv_bfloat16*)dy, dwte, dwpe, T, S, D, V);
  CHECK_LAUNCH();
}
extern "C" int inv_colsum(const void* x, float* out, int T, int N, int ld, void* stream) {
  if (N % 2 || ld % 2) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  if (N % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int gx = (N + 255) / 256;
    int chunks = (148 * 4 + gx - 1) / gx;          // four CTAs per SM over the whole grid
    const int max_chunks = (T + 63) / 64;          // at least 64 rows (8 per warp) per CTA
    if (chunks > max_chunks) chunks = max_chunks;
    const int rows_per_block = (T + chunks - 1) / chunks;
    colsum_kernel<<<dim3(gx, chunks), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, out, T, N, ld, rows_per_block);
    CHECK_LAUNCH();
  }
  int chunks = (T + 2047) / 2048;
  if (chunks > 64) chunks = 64;
  const int rows_per_block = (T + chunks - 1) / chunks;
  dim3 grid((N + 63) / 64, chunks);
  colsum2_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, out, T, N, ld, rows_per_block);
  CHECK_LAUNCH();
}
extern "C" int inv_act(const void* x, const void* dy, void* out, long rows, int F, int mode, void* stream) {
  if (F % 8) return -ERR_BAD_ARG;
  if (rows <= 0) return 0;
  act_kernel<<<grid_for(rows * F / 8, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                          (__nv_bfloat16*)out, rows, F, mode, nullptr);
  CHECK_LAUNCH();
}
// The same over the first min(max_rows, *rows_dev) rows: buffers sized for a capacity, filled to a count known on the device.
extern "C" int inv_act_rows(const void* x, const void* dy, void* out, long max_rows, const int* rows_dev, int F, int mode, void* stream) {
  if (F % 8 || rows_dev == nullptr) return -ERR_BAD_ARG;
  if (max_rows <= 0) return 0;
  long blocks = (max_rows * (F / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  act_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)out, max_rows, F,
                                                            mode, rows_dev);
  CHECK_LAUNCH();
}
extern "C" int inv_rope(void* buf, const int* pos, const float* cos_t, const float* sin_t, int T, int S, int ld, int col0, int nheads, int hd,
                        int inverse, void* stream) {
  if (hd % 16 || ld % 8 || col0 % 8) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  rope_kernel<<<grid_for((long)T * nheads * hd / 16, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)buf, pos, cos_t, sin_t, T, S, ld,
                                                                                         col0, nheads, hd, inverse);
  CHECK_LAUNCH();
}
extern "C" int inv_add(const void* a, const void* b, void* y, long n, void* stream) {
  if (n % 8) return -ERR_BAD_ARG;
  if (n <= 0) return 0;
  add_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n / 8);
  CHECK_LAUNCH();
}
extern "C" int inv_l2_flush(void* buf, long bytes, void* stream) {
  l2_flush_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>((uint4*)buf, bytes / 16);
  CHECK_LAUNCH();
}
