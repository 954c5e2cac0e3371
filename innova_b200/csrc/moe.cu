// Mixture-of-experts routing, dispatch and combine.
//
// Replaces the reference's softmax_with_topk (src/moe_variants.cpp:97-138: full softmax over the
// experts, top-k by value, weights are the raw probabilities), compute_load_balance_loss and the
// z-loss (src/moe_variants.cpp:140-175), moe_dispatch_batched (src/moe_variants.cpp:767-829: group
// tokens per expert, expert FFN, weighted scatter-add) and the moe_gather / moe_scatter_add shaders
// (src/gpu_compute.cpp:151-176).
//
// Layout: tokens routed to expert e occupy rows [offset[e], offset[e] + count[e]) of the permuted
// buffer; every segment starts on a multiple of 128 rows so that a 128-row GEMM tile belongs to one
// expert and a 64-token k-block of the weight-gradient GEMM never straddles two experts. Padding rows
// are zero. `slot[t, k]` remembers where token t's k-th choice went, which is all that combine and
// the backward passes need.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {

constexpr int MOE_ALIGN = 128;
constexpr int MOE_MAX_E = 64;

// One warp per token. logits [T, E] fp32. Outputs: probs [T, E] fp32 (softmax), topk_idx / topk_w
// [T, K], counts[E] (+= 1 per routed token), stats[0..E) += probability mass per expert,
// stats[E..2E) += logit mass of the selected experts (the reference's load-balance term),
// stats[2E] += sum of logsumexp^2 (z-loss).
__global__ void __launch_bounds__(256) moe_router_kernel(const float* __restrict__ logits, float* __restrict__ probs, int* __restrict__ topk_idx,
                                                         float* __restrict__ topk_w, int* __restrict__ counts, float* __restrict__ stats, int T,
                                                         int E, int K) {
  __shared__ float s_stats[2 * MOE_MAX_E + 1];
  __shared__ int s_counts[MOE_MAX_E];
  for (int i = threadIdx.x; i < 2 * E + 1; i += blockDim.x) s_stats[i] = 0.f;
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_counts[i] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t < T) {
    const float l0 = lane < E ? logits[(size_t)t * E + lane] : -INFINITY;
    const float l1 = lane + 32 < E ? logits[(size_t)t * E + lane + 32] : -INFINITY;
    float mx = fmaxf(l0, l1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float e0 = lane < E ? __expf(l0 - mx) : 0.f, e1 = lane + 32 < E ? __expf(l1 - mx) : 0.f;
    float z = e0 + e1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    const float p0 = e0 / z, p1 = e1 / z;
    if (lane < E) {
      probs[(size_t)t * E + lane] = p0;
      atomicAdd(&s_stats[lane], p0);
    }
    if (lane + 32 < E) {
      probs[(size_t)t * E + lane + 32] = p1;
      atomicAdd(&s_stats[lane + 32], p1);
    }
    if (lane == 0) {
      const float lse = mx + __logf(z);
      atomicAdd(&s_stats[2 * E], lse * lse);
    }
    float c0 = p0, c1 = p1;  // candidates; taken ones become -1
    if (lane >= E) c0 = -1.f;
    if (lane + 32 >= E) c1 = -1.f;
    for (int k = 0; k < K; ++k) {
      float best = c0 >= c1 ? c0 : c1;
      int bi = c0 >= c1 ? lane : lane + 32;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) {
          best = ob;
          bi = oi;
        }
      }
      if (lane == 0) {
        topk_idx[(size_t)t * K + k] = bi;
        topk_w[(size_t)t * K + k] = best;
        atomicAdd(&s_counts[bi], 1);
      }
      if (bi == lane) {
        atomicAdd(&s_stats[E + bi], l0);
        c0 = -1.f;
      }
      if (bi == lane + 32) {
        atomicAdd(&s_stats[E + bi], l1);
        c1 = -1.f;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * E + 1; i += blockDim.x)
    if (s_stats[i] != 0.f) atomicAdd(&stats[i], s_stats[i]);
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (s_counts[i]) atomicAdd(&counts[i], s_counts[i]);
}

// counts[E] -> offsets[E+1] (segment starts, multiples of 128; offsets[E] = rows used),
// tile_expert[max_tiles] (expert of each 128-row tile, -1 beyond the last), cursor[E] = 0.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ tile_expert,
                                   int* __restrict__ cursor, int E, int max_tiles) {
  __shared__ int s_off[MOE_MAX_E + 1];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = run;
      run += (counts[e] + MOE_ALIGN - 1) / MOE_ALIGN * MOE_ALIGN;
    }
    s_off[E] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < E) cursor[e] = 0;
  }
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * MOE_ALIGN;
    int ex = -1;
    for (int e = 0; e < E; ++e)
      if (row >= s_off[e] && row < s_off[e + 1]) ex = e;
    tile_expert[t] = ex;
  }
}

// One warp per (token, choice): claims a slot in its expert's segment and copies the token's row there.
// scale_w != nullptr multiplies the row by topk weight (used by the combine backward).
__global__ void __launch_bounds__(256) moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                                                          const int* __restrict__ offsets, int* __restrict__ cursor, int* __restrict__ slot,
                                                          const float* __restrict__ scale_w, __nv_bfloat16* __restrict__ x_perm, int T, int K,
                                                          int D, int assign) {
  const int lane = threadIdx.x & 31;
  const long id = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long)T * K) return;
  const int t = (int)(id / K);
  int s;
  if (assign) {
    if (lane == 0) {
      const int e = topk_idx[id];
      s = offsets[e] + atomicAdd(&cursor[e], 1);
      slot[id] = s;
    }
    s = __shfl_sync(0xffffffffu, s, 0);
  } else {
    s = slot[id];
  }
  const float w = scale_w ? scale_w[id] : 1.f;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * D);
  uint4* dst = reinterpret_cast<uint4*>(x_perm + (size_t)s * D);
  for (int i = lane; i < D / 8; i += 32) {
    uint4 v = src[i];
    if (scale_w) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(f.x * w, f.y * w);
      }
    }
    dst[i] = v;
  }
}

// out[t] = sum_k w[t,k] * y_perm[slot[t,k]] (+ residual[t]).  One warp per token.
// If dw != nullptr it also produces dw[t,k] = <y_perm[slot[t,k]], g[t]> (gradient of the routing weights),
// in which case `weights` may be null (plain sum: gathers dx from the permuted gradient).
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y_perm, const int* __restrict__ slot,
                                                          const float* __restrict__ weights, const __nv_bfloat16* __restrict__ residual,
                                                          __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ g,
                                                          float* __restrict__ dw, int T, int K, int D) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  for (int i = lane; i < D / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (residual) {
      const uint4 r = reinterpret_cast<const uint4*>(residual + (size_t)t * D)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int k = 0; k < K; ++k) {
      const int s = slot[(size_t)t * K + k];
      const float w = weights ? weights[(size_t)t * K + k] : 1.f;
      const uint4 v = reinterpret_cast<const uint4*>(y_perm + (size_t)s * D)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += w * f.x;
        acc[2 * j + 1] += w * f.y;
      }
    }
    if (out) {
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + (size_t)t * D)[i] = o;
    }
  }
  if (dw) {
    for (int k = 0; k < K; ++k) {
      const int s = slot[(size_t)t * K + k];
      float d = 0.f;
      for (int i = lane; i < D / 8; i += 32) {
        const uint4 v = reinterpret_cast<const uint4*>(y_perm + (size_t)s * D)[i];
        const uint4 gg = reinterpret_cast<const uint4*>(g + (size_t)t * D)[i];
        const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&v);
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&gg);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __bfloat1622float2(a[j]), fb = __bfloat1622float2(b[j]);
          d += fa.x * fb.x + fa.y * fb.y;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (lane == 0) dw[(size_t)t * K + k] = d;
    }
  }
}

}  // namespace inv

using namespace inv;
#define MOE_RET()                           \
  do {                                      \
    cudaError_t e = cudaGetLastError();     \
    return e == cudaSuccess ? 0 : -(int)e;  \
  } while (0)

extern "C" int inv_moe_router(const float* logits, float* probs, int* topk_idx, float* topk_w, int* counts, float* stats, int T, int E, int K,
                              void* stream) {
  if (E < 1 || E > MOE_MAX_E || K < 1 || K > E) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  moe_router_kernel<<<(T + 7) / 8, 256, 0, (cudaStream_t)stream>>>(logits, probs, topk_idx, topk_w, counts, stats, T, E, K);
  MOE_RET();
}
extern "C" int inv_moe_offsets(const int* counts, int* offsets, int* tile_expert, int* cursor, int E, int max_tiles, void* stream) {
  if (E < 1 || E > MOE_MAX_E) return -ERR_BAD_ARG;
  moe_offsets_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(counts, offsets, tile_expert, cursor, E, max_tiles);
  MOE_RET();
}
extern "C" int inv_moe_scatter(const void* x, const int* topk_idx, const int* offsets, int* cursor, int* slot, const float* scale_w, void* x_perm,
                               int T, int K, int D, int assign, void* stream) {
  if (D % 8) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  const long warps = (long)T * K;
  moe_scatter_kernel<<<(int)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, topk_idx, offsets, cursor, slot, scale_w,
                                                                              (__nv_bfloat16*)x_perm, T, K, D, assign);
  MOE_RET();
}
extern "C" int inv_moe_combine(const void* y_perm, const int* slot, const float* weights, const void* residual, void* out, const void* g, float* dw,
                               int T, int K, int D, void* stream) {
  if (D % 8) return -ERR_BAD_ARG;
  if (T <= 0) return 0;
  moe_combine_kernel<<<(T + 7) / 8, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)y_perm, slot, weights, (const __nv_bfloat16*)residual,
                                                                   (__nv_bfloat16*)out, (const __nv_bfloat16*)g, dw, T, K, D);
  MOE_RET();
}
