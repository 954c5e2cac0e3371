// LayerNorm and RMSNorm, forward and backward, bf16 activations with fp32 statistics.
//
// Replaces the reference's math::layer_norm / layer_norm_grad (src/math_avx2.cpp:349-412,
// src/autograd_grad.cpp:142-181), math::rms_norm / rms_norm_grad (src/math_avx2.cpp:414-457,
// src/autograd_grad.cpp:183-218) and the fused residual-add RMSNorm (src/gpu_compute_vulkan.cpp:1232-1245).
//
// One warp owns one row and reads it with 16-byte loads (8 bf16). Re-reads of a row hit L1. The
// backward kernels are persistent; each CTA keeps its share of the gamma/beta gradient on chip and
// writes one partial row per CTA to a scratch buffer [grid, 2, D] (fp32) that a second kernel folds
// into the fp32 gradient (+=).
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// ----------------------------------------------------------------------------------------------
// Forward. RMS = true: y = x * rsqrt(mean(x^2) + eps) * gamma. Otherwise LayerNorm with beta.
// If `res` is given, the row normalised is x + res and `xsum` receives that sum (residual stream).
// ----------------------------------------------------------------------------------------------
template <bool RMS>
__global__ void __launch_bounds__(256) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                                       const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                                                       __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ xsum,
                                                       float* __restrict__ mean_out, float* __restrict__ rstd_out, int T, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (row >= T) return;
  const __nv_bfloat16* xr = x + (size_t)row * D;
  const __nv_bfloat16* rr = res ? res + (size_t)row * D : nullptr;
  float s = 0.f;
  if (rr) {
    __nv_bfloat16* xs = xsum + (size_t)row * D;
    for (int c = lane * 8; c < D; c += 256) {
      float a[8], b[8];
      load8(xr + c, a);
      load8(rr + c, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
      store8(xs + c, a);
      // statistics use the rounded sum so that backward sees the same row
      float t[8];
      load8(xs + c, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += RMS ? t[j] * t[j] : t[j];
    }
    xr = xs;
  } else {
    for (int c = lane * 8; c < D; c += 256) {
      float a[8];
      load8(xr + c, a);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += RMS ? a[j] * a[j] : a[j];
    }
  }
  s = warp_sum(s);
  float mean = 0.f, rstd;
  if (RMS) {
    rstd = rsqrtf(s / D + eps);
  } else {
    mean = s / D;
    float v = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      float a[8];
      load8(xr + c, a);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float d = a[j] - mean;
        v += d * d;
      }
    }
    v = warp_sum(v);
    rstd = rsqrtf(v / D + eps);
  }
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  __nv_bfloat16* yr = y + (size_t)row * D;
  for (int c = lane * 8; c < D; c += 256) {
    float a[8], g[8], o[8];
    load8(xr + c, a);
    load8(gamma + c, g);
    if (!RMS && beta) {
      float b[8];
      load8(beta + c, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (a[j] - mean) * rstd * g[j] + b[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (a[j] - mean) * rstd * g[j];
    }
    store8(yr + c, o);
  }
}

// Forward for D <= 1024: the row is read once into packed registers (the next row of the warp is in flight meanwhile),
// mean and variance are two passes over registers, not over memory. Persistent grid: a warp walks rows gw, gw + nw, ...
template <bool RMS, int NCH>
__global__ void __launch_bounds__(256) norm_fwd_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                                            const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                                                            __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ xsum,
                                                            float* __restrict__ mean_out, float* __restrict__ rstd_out, int T, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int gw = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int nw = gridDim.x * 8;
  uint4 gp[NCH], bp[NCH];
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = k * 256 + lane * 8;
    gp[k] = bp[k] = make_uint4(0, 0, 0, 0);
    if (c < D) {
      gp[k] = *reinterpret_cast<const uint4*>(gamma + c);
      if (!RMS && beta) bp[k] = *reinterpret_cast<const uint4*>(beta + c);
    }
  }
  uint4 nx[NCH], nr[NCH];
  auto fetch = [&](int row) {
    if (row >= T) return;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < D) {
        nx[k] = *reinterpret_cast<const uint4*>(x + (size_t)row * D + c);
        if (res) nr[k] = *reinterpret_cast<const uint4*>(res + (size_t)row * D + c);
      }
    }
  };
  fetch(gw);
  for (int row = gw; row < T; row += nw) {
    float v[NCH][8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < D) {
        unpack8(nx[k], v[k]);
        if (res) {
          float r[8];
          unpack8(nr[k], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[k][j] += r[j];
          // the residual stream is stored rounded, and the statistics use the rounded sum so that backward sees the same row
          uint4 packed;
          packed.x = pack_bf16x2(v[k][0], v[k][1]);
          packed.y = pack_bf16x2(v[k][2], v[k][3]);
          packed.z = pack_bf16x2(v[k][4], v[k][5]);
          packed.w = pack_bf16x2(v[k][6], v[k][7]);
          *reinterpret_cast<uint4*>(xsum + (size_t)row * D + c) = packed;
          unpack8(packed, v[k]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s += RMS ? v[k][j] * v[k][j] : v[k][j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[k][j] = 0.f;
      }
    }
    fetch(row + nw);
    s = warp_sum(s);
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(s / D + eps);
    } else {
      mean = s / D;
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = k * 256 + lane * 8;
        if (c < D) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float d = v[k][j] - mean;
            q += d * d;
          }
        }
      }
      q = warp_sum(q);
      rstd = rsqrtf(q / D + eps);
    }
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < D) {
        float g[8], b[8], o[8];
        unpack8(gp[k], g);
        unpack8(bp[k], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[k][j] - mean) * rstd * g[j] + b[j];
        store8(y + (size_t)row * D + c, o);
      }
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Backward. dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) for LayerNorm (g = dy * gamma),
// dx = rstd * (g - xhat * mean(g * xhat)) for RMSNorm. If `dres` is given it is added to dx
// (gradient arriving on the residual stream). Per-CTA partial dgamma/dbeta go to `partial`.
// ----------------------------------------------------------------------------------------------
template <bool RMS>
__global__ void __launch_bounds__(256) norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                       const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                                                       const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                                                       __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int T, int D) {
  // [2][Dp]: dgamma, dbeta. Column c lives at slot(c), which spreads the 8 columns a lane owns
  // over 8 different 32-float rows so that a warp's atomics fall into 32 distinct banks.
  extern __shared__ float acc[];
  const int Dp = (D + 255) & ~255;
  for (int i = threadIdx.x; i < 2 * Dp; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int gw = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int nw = gridDim.x * warps_per_block;
  for (int row = gw; row < T; row += nw) {
    const __nv_bfloat16* xr = x + (size_t)row * D;
    const __nv_bfloat16* dyr = dy + (size_t)row * D;
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      float a[8], d[8], g[8];
      load8(xr + c, a);
      load8(dyr + c, d);
      load8(gamma + c, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float xh = (a[j] - mean) * rstd;
        float gg = d[j] * g[j];
        s1 += gg;
        s2 += gg * xh;
      }
    }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
    if (RMS) s1 = 0.f;
    __nv_bfloat16* dxr = dx + (size_t)row * D;
    const __nv_bfloat16* drr = dres ? dres + (size_t)row * D : nullptr;
    for (int c = lane * 8; c < D; c += 256) {
      float a[8], d[8], g[8], o[8];
      load8(xr + c, a);
      load8(dyr + c, d);
      load8(gamma + c, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float xh = (a[j] - mean) * rstd;
        o[j] = rstd * (d[j] * g[j] - s1 - xh * s2);
        const int slot = (c & ~255) + j * 32 + lane;
        atomicAdd(&acc[slot], d[j] * xh);
        if (!RMS) atomicAdd(&acc[Dp + slot], d[j]);
      }
      if (drr) {
        float r[8];
        load8(drr + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      store8(dxr + c, o);
    }
  }
  __syncthreads();
  float* out = partial + (size_t)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
    const int col = i < D ? i : i - D;
    const int slot = (col & ~255) + (col & 7) * 32 + ((col & 255) >> 3);
    out[i] = acc[(i < D ? 0 : Dp) + slot];
  }
}


// ----------------------------------------------------------------------------------------------
// Backward for D <= 1024, the bandwidth-bound form. A warp owns a row; the x and dy of the next TWO rows of the warp are
// in flight as packed registers while the current row is reduced and written (one row ahead left the memory system
// under-subscribed: 8 warps per SM with 4.6 KB each). The row is unpacked twice (sums, then dx) instead of being held in
// fp32. CS adds a third column sum next to dgamma / dbeta: the column sums of the dx that is written, which is the bias
// gradient of the linear layer that feeds the residual stream at this point.
// ----------------------------------------------------------------------------------------------
template <bool RMS, int NCH, bool CS>
__global__ void __launch_bounds__(256, 1) norm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                                                               const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                                                               __nv_bfloat16* __restrict__ dx, float* __restrict__ partial,
                                                               float* __restrict__ partial_cs, int T, int D) {
  __shared__ float red[8][256];  // one 256-column slab at a time
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gw = blockIdx.x * 8 + warp;
  const int nw = gridDim.x * 8;
  float g[NCH][8], dg[NCH][8], db[NCH][8], dc[CS ? NCH : 1][8];
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = k * 256 + lane * 8;
    if (c < D) load8(gamma + c, g[k]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[k][j] = 0.f;
      db[k][j] = 0.f;
      if (CS) dc[k][j] = 0.f;
      if (c >= D) g[k][j] = 0.f;
    }
  }
  struct Row {
    uint4 x[NCH], d[NCH];
    float mean, rstd;
  };
  auto fetch = [&](int row, Row& R) {
    if (row >= T) return;
    const __nv_bfloat16* xr = x + (size_t)row * D;
    const __nv_bfloat16* dyr = dy + (size_t)row * D;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < D) {
        R.x[k] = *reinterpret_cast<const uint4*>(xr + c);
        R.d[k] = *reinterpret_cast<const uint4*>(dyr + c);
      }
    }
    R.mean = RMS ? 0.f : mean_in[row];
    R.rstd = rstd_in[row];
  };
  auto process = [&](int row, const Row& R) {
    uint4 rr[NCH];
    if (dres) {
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = k * 256 + lane * 8;
        if (c < D) rr[k] = *reinterpret_cast<const uint4*>(dres + (size_t)row * D + c);
      }
    }
    const float mean = R.mean, rstd = R.rstd;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < D) {
        float xv[8], dv[8];
        unpack8(R.x[k], xv);
        unpack8(R.d[k], dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gg = dv[j] * g[k][j];
          s1 += gg;
          s2 += gg * ((xv[j] - mean) * rstd);
        }
      }
    }
    s1 = RMS ? 0.f : warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
    __nv_bfloat16* dxr = dx + (size_t)row * D;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < D) {
        float xv[8], dv[8], o[8];
        unpack8(R.x[k], xv);
        unpack8(R.d[k], dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          o[j] = rstd * (dv[j] * g[k][j] - s1 - xh * s2);
          dg[k][j] += dv[j] * xh;
          db[k][j] += dv[j];
        }
        if (dres) {
          float r[8];
          unpack8(rr[k], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        if (CS) {
#pragma unroll
          for (int j = 0; j < 8; ++j) dc[k][j] += o[j];
        }
        store8(dxr + c, o);
      }
    }
  };
  if constexpr (NCH <= 3) {  // two rows ahead
    Row r0, r1, r2;
    fetch(gw, r0);
    fetch(gw + nw, r1);
    for (int row = gw; row < T; row += 3 * nw) {
      fetch(row + 2 * nw, r2);
      process(row, r0);
      if (row + nw < T) {
        fetch(row + 3 * nw, r0);
        process(row + nw, r1);
      }
      if (row + 2 * nw < T) {
        fetch(row + 4 * nw, r1);
        process(row + 2 * nw, r2);
      }
    }
  } else {  // 769 .. 1024 columns: the register file holds one row ahead
    Row r0, r1;
    fetch(gw, r0);
    for (int row = gw; row < T; row += 2 * nw) {
      fetch(row + nw, r1);
      process(row, r0);
      if (row + nw < T) {
        fetch(row + 2 * nw, r0);
        process(row + nw, r1);
      }
    }
  }
  // fold the 8 warps of the CTA, one 256-column slab at a time, and write this CTA's partial rows
  float* out = partial + (size_t)blockIdx.x * 2 * D;
#pragma unroll
  for (int which = 0; which < (CS ? 3 : 2); ++which) {
    if (RMS && which == 1) continue;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = which == 0 ? dg[k][j] : which == 1 ? db[k][j] : dc[CS ? k : 0][j];
      __syncthreads();
      const int c = k * 256 + threadIdx.x;
      if (c < D) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
        if (which < 2) out[which * D + c] = s;
        else partial_cs[(size_t)blockIdx.x * D + c] = s;
      }
    }
  }
  if (RMS) {
    for (int c = threadIdx.x; c < D; c += 256) out[D + c] = 0.f;
  }
}

// dgamma[D] += sum_b partial[b][0][:], dbeta[D] += sum_b partial[b][1][:], colsum[D] = sum_b partial_cs[b][:].
// grid (ceil(D / 32), 3): a CTA owns 32 columns of one of the three sums; its 8 warps take the partial rows round robin
// (coalesced 128-byte reads) and meet in shared memory.
__global__ void __launch_bounds__(256) norm_bwd_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ partial_cs,
                                                              float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                              float* __restrict__ colsum, int nblocks, int D) {
  __shared__ float red[8][32];
  const int which = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float* dst = which == 0 ? dgamma : which == 1 ? dbeta : colsum;
  if (dst == nullptr) return;
  float s = 0.f;
  if (c < D) {
    if (which < 2) {
      for (int b = warp; b < nblocks; b += 8) s += partial[(size_t)b * 2 * D + which * D + c];
    } else {
      for (int b = warp; b < nblocks; b += 8) s += partial_cs[(size_t)b * D + c];
    }
  }
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < D) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][lane];
    if (which < 2) dst[c] += t;
    else dst[c] = t;
  }
}

}  // namespace inv

using namespace inv;

extern "C" int inv_norm_fwd(const void* x, const void* res, const void* gamma, const void* beta, void* y, void* xsum, float* mean,
                            float* rstd, int T, int D, float eps, int rms, void* stream) {
  if (D % 8) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int wpb = 8;
  dim3 grid((T + wpb - 1) / wpb), block(wpb * 32);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<const __nv_bfloat16*>(res);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto B = reinterpret_cast<const __nv_bfloat16*>(beta);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  auto XS = reinterpret_cast<__nv_bfloat16*>(xsum);
  const int nch = (D + 255) / 256;
  if (nch <= 4) {  // register path, persistent grid
    int g = (T + 7) / 8;
    if (g > 148 * 2) g = 148 * 2;  // two CTAs per SM at 124 registers: one resident wave
#define INV_NF_ROWS(R_, N_) norm_fwd_rows_kernel<R_, N_><<<g, 256, 0, st>>>(X, R, G, B, Y, XS, mean, rstd, T, D, eps)
    if (rms) {
      if (nch == 1) INV_NF_ROWS(true, 1); else if (nch == 2) INV_NF_ROWS(true, 2); else if (nch == 3) INV_NF_ROWS(true, 3); else INV_NF_ROWS(true, 4);
    } else {
      if (nch == 1) INV_NF_ROWS(false, 1); else if (nch == 2) INV_NF_ROWS(false, 2); else if (nch == 3) INV_NF_ROWS(false, 3); else INV_NF_ROWS(false, 4);
    }
#undef INV_NF_ROWS
  } else if (rms) norm_fwd_kernel<true><<<grid, block, 0, st>>>(X, R, G, B, Y, XS, mean, rstd, T, D, eps);
  else norm_fwd_kernel<false><<<grid, block, 0, st>>>(X, R, G, B, Y, XS, mean, rstd, T, D, eps);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// Number of CTAs the backward launches for T rows; scratch must hold grid * 3 * D floats (2 * D per CTA for dgamma and
// dbeta, then D per CTA for the optional column sums of dx).
extern "C" int inv_norm_bwd_grid(int T) {
  int g = (T + 7) / 8;
  return g < 148 ? (g < 1 ? 1 : g) : 148;
}

// colsum (nullable, D <= 1024 only): fp32 [D], overwritten with the column sums of dx as written (dres included).
static int norm_bwd_launch(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres, void* dx,
                           float* dgamma, float* dbeta, float* colsum, float* scratch, int grid, int T, int D, int rms, cudaStream_t st) {
  const size_t smem = (size_t)2 * ((D + 255) & ~255) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(norm_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 12288 * 4);
    cudaFuncSetAttribute(norm_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 12288 * 4);
    configured = true;
  }
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto DR = reinterpret_cast<const __nv_bfloat16*>(dres);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  const int nch = (D + 255) / 256;
  float* scratch_cs = scratch + (size_t)grid * 2 * D;
  if (colsum != nullptr && nch > 4) return -ERR_BAD_ARG;
#define INV_NB_ROWS(R, N)                                                                                                             \
  do {                                                                                                                                \
    if (colsum) norm_bwd_rows_kernel<R, N, true><<<grid, 256, 0, st>>>(DY, X, G, mean, rstd, DR, DX, scratch, scratch_cs, T, D);      \
    else norm_bwd_rows_kernel<R, N, false><<<grid, 256, 0, st>>>(DY, X, G, mean, rstd, DR, DX, scratch, scratch_cs, T, D);            \
  } while (0)
  if (nch <= 4) {  // register path
    if (rms) {
      if (nch == 1) INV_NB_ROWS(true, 1); else if (nch == 2) INV_NB_ROWS(true, 2); else if (nch == 3) INV_NB_ROWS(true, 3); else INV_NB_ROWS(true, 4);
    } else {
      if (nch == 1) INV_NB_ROWS(false, 1); else if (nch == 2) INV_NB_ROWS(false, 2); else if (nch == 3) INV_NB_ROWS(false, 3); else INV_NB_ROWS(false, 4);
    }
  } else if (rms) {
    norm_bwd_kernel<true><<<grid, 256, smem, st>>>(DY, X, G, mean, rstd, DR, DX, scratch, T, D);
  } else {
    norm_bwd_kernel<false><<<grid, 256, smem, st>>>(DY, X, G, mean, rstd, DR, DX, scratch, T, D);
  }
#undef INV_NB_ROWS
  norm_bwd_reduce_kernel<<<dim3((D + 31) / 32, colsum ? 3 : 2), 256, 0, st>>>(scratch, scratch_cs, dgamma, rms ? nullptr : dbeta, colsum, grid, D);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres,
                            void* dx, float* dgamma, float* dbeta, float* scratch, int T, int D, int rms, void* stream) {
  if (D % 8 || D > 12288) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  return norm_bwd_launch(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, nullptr, scratch, inv_norm_bwd_grid(T), T, D, rms,
                         reinterpret_cast<cudaStream_t>(stream));
}

// The same with the column sums of dx (fp32 [D], overwritten) as a by-product: D <= 1024.
extern "C" int inv_norm_bwd_colsum(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres,
                                   void* dx, float* dgamma, float* dbeta, float* colsum, float* scratch, int T, int D, int rms, void* stream) {
  if (D % 8 || D > 1024 || colsum == nullptr) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  return norm_bwd_launch(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, colsum, scratch, inv_norm_bwd_grid(T), T, D, rms,
                         reinterpret_cast<cudaStream_t>(stream));
}

// ----------------------------------------------------------------------------------------------
// No-allocation variant of the backward (declared and documented in inv_noalloc.h).
// The partial sums go to a file-scope device array instead of caller-provided scratch. In host code
// the array's name is only a handle: its device address comes from cudaGetSymbolAddress, looked up
// once per device with that device current, and that address is what the kernels receive.
// ----------------------------------------------------------------------------------------------
#include "inv_noalloc.h"

#include <mutex>

static __device__ __align__(256) float g_norm_bwd_partials[INV_NOALLOC_NORM_MAX_GRID * 2 * INV_NOALLOC_NORM_MAX_D];

namespace {
constexpr int kMaxDevices = 64;
float* g_partials_addr[kMaxDevices] = {nullptr};
std::mutex g_partials_mutex;

// Device address of the static array on the current device, or nullptr with *err set.
float* noalloc_partials(cudaError_t* err) {
  int dev = -1;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= kMaxDevices) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_partials_mutex);
  if (g_partials_addr[dev] == nullptr) {
    void* p = nullptr;
    *err = cudaGetSymbolAddress(&p, g_norm_bwd_partials);
    if (*err != cudaSuccess) return nullptr;
    g_partials_addr[dev] = static_cast<float*>(p);
  }
  return g_partials_addr[dev];
}
}  // namespace

extern "C" int inv_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres,
                                    void* dx, float* dgamma, float* dbeta, int T, int D, int rms, void* stream) {
  if (D <= 0 || (D % 8) != 0 || D > INV_NOALLOC_NORM_MAX_D) return -ERR_BAD_ARG;  // beyond the static scratch
  if (T <= 0) return 0;
  cudaError_t err = cudaSuccess;
  float* partials = noalloc_partials(&err);
  if (partials == nullptr) return -(int)err;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int grid = (T + 7) / 8;
  if (grid > INV_NOALLOC_NORM_MAX_GRID) grid = INV_NOALLOC_NORM_MAX_GRID;
  const size_t smem = (size_t)2 * ((D + 255) & ~255) * sizeof(float);  // at most 16 KiB: no opt-in needed
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto DR = reinterpret_cast<const __nv_bfloat16*>(dres);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  if (rms) norm_bwd_kernel<true><<<grid, 256, smem, st>>>(DY, X, G, mean, rstd, DR, DX, partials, T, D);
  else norm_bwd_kernel<false><<<grid, 256, smem, st>>>(DY, X, G, mean, rstd, DR, DX, partials, T, D);
  norm_bwd_reduce_kernel<<<dim3((D + 31) / 32, 2), 256, 0, st>>>(partials, nullptr, dgamma, rms ? nullptr : dbeta, nullptr, grid, D);
  err = cudaGetLastError();
  return err == cudaSuccess ? 0 : -(int)err;
}
