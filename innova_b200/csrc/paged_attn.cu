// Paged KV cache on the device: append (with OIL4 quantisation) and single-query decode attention.
//
// Replaces the reference's PagedAttention::forward (src/inference_opt.cpp:60-112: block-table walk
// with online softmax per query row), the OIL4 KV cache (src/kv_cache_oil4.cpp:207-362) and the
// int8 block KV quantiser (src/kv_cache.cpp:15-44). The reference fits a 16-entry Lloyd codebook per
// block on the CPU at append time; here every block of 32 values stores an fp16 abs-max scale and
// 4-bit indices into one fixed 16-level Gaussian codebook, which a GPU can produce at append time
// without iterations and read back with a 16-entry register LUT.
//
// Pools (page = 16 tokens): KV_OIL4: idx [pages, Hkv, 16, D/2] bytes, scale [pages, Hkv, 16, D/32] fp16.
//                           KV_BF16: data [pages, Hkv, 16, D] bf16 (scale pool unused).
// page_table [B, max_pages] int32 maps a sequence's logical page to a pool page.
#include "sm100_common.cuh"
#include "inv_api.h"

#include <cuda_fp16.h>

namespace inv {

constexpr int PAGE = 16;
__constant__ float c_kv_levels[16] = {-1.0f, -0.755096f, -0.588527f, -0.455957f, -0.341269f, -0.239458f, -0.146295f, -0.046361f,
                                      0.046361f, 0.146295f, 0.239458f, 0.341269f, 0.455957f, 0.588527f, 0.755096f, 1.0f};

__device__ __forceinline__ int nearest_level16(float x) {
  int lo = 0;
#pragma unroll
  for (int step = 8; step > 0; step >>= 1)
    if (c_kv_levels[lo + step] <= x) lo += step;
  if (lo < 15 && (c_kv_levels[lo + 1] - x) < (x - c_kv_levels[lo])) ++lo;
  return lo;
}

// One warp per (token, kv head, k-or-v): lane handles D/32 consecutive... each lane owns the elements
// e = lane + 32*j (one per 32-block j), so a block's abs-max is a warp reduction and nibble pairs are
// formed with a shuffle.
template <bool OIL4>
__global__ void __launch_bounds__(256) kv_append_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new, int ld_k,
                                                        int ld_v, const int* __restrict__ page_table, int max_pages,
                                                        const int* __restrict__ start_pos, int B, int S_new, int Hkv, int D,
                                                        uint8_t* __restrict__ k_pool, uint8_t* __restrict__ v_pool, __half* __restrict__ k_scale,
                                                        __half* __restrict__ v_scale) {
  const int lane = threadIdx.x & 31;
  const long warp_id = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const long total = (long)B * S_new * Hkv * 2;
  if (warp_id >= total) return;
  const int which = (int)(warp_id & 1);
  long r = warp_id >> 1;
  const int hk = (int)(r % Hkv);
  r /= Hkv;
  const int s = (int)(r % S_new);
  const int b = (int)(r / S_new);
  const int pos = start_pos[b] + s;
  const int page = page_table[(long)b * max_pages + pos / PAGE];
  const int slot = pos % PAGE;
  const __nv_bfloat16* src = (which ? v_new : k_new) + ((long)b * S_new + s) * (which ? ld_v : ld_k) + hk * D;
  uint8_t* pool = which ? v_pool : k_pool;
  const long row = ((long)page * Hkv + hk) * PAGE + slot;
  if (!OIL4) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(pool) + row * D;
    for (int e = lane; e < D; e += 32) dst[e] = src[e];
    return;
  }
  __half* sc = (which ? v_scale : k_scale) + row * (D / 32);
  uint8_t* dst = pool + row * (D / 2);
  for (int j = 0; j < D / 32; ++j) {
    const float w = __bfloat162float(src[j * 32 + lane]);
    float amax = fabsf(w);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax < 1e-10f ? 1.f : amax;
    const int code = nearest_level16(w / scale);
    const int hi = __shfl_down_sync(0xffffffffu, code, 1);
    if ((lane & 1) == 0) dst[j * 16 + (lane >> 1)] = (uint8_t)(code | (hi << 4));
    if (lane == 0) sc[j] = __float2half_rn(scale);
  }
}

// Rows of a token tree. Without it, query row b is the newest token of sequence b and sees seq_lens[b] cached tokens.
// With it, query row b belongs to sequence row_seq[b] (several rows may share one), sees every cached token below
// tail_start[b], and of the at most 64 tokens from tail_start[b] on only those whose bit is set in tail_mask[b]
// (its ancestors in the tree and itself). All three pointers are null or all are set.
struct TreeRows {
  const int* row_seq;
  const int* tail_start;
  const unsigned long long* tail_mask;
};
__device__ __forceinline__ bool token_visible(int tok, int len, int tail0, unsigned long long tail_bits) {
  return tok < len && (tok < tail0 || ((tail_bits >> ((tok - tail0) & 63)) & 1ull));
}

// Decode attention: one query token per sequence. grid = (splits, Hkv, B), 128 threads.
// Writes partial (m, l, o[G][D]) per (b, hk, split) to scratch; attn_combine_kernel finishes.
template <bool OIL4, int D>
__global__ void __launch_bounds__(128) paged_decode_kernel(const __nv_bfloat16* __restrict__ q, int ld_q, const int* __restrict__ page_table,
                                                           int max_pages, const int* __restrict__ seq_lens, int H, int Hkv,
                                                           const uint8_t* __restrict__ k_pool, const uint8_t* __restrict__ v_pool,
                                                           const __half* __restrict__ k_scale, const __half* __restrict__ v_scale, float scale,
                                                           float* __restrict__ part, int splits, TreeRows tree) {
  constexpr int MAXG = 8;
  constexpr int EPL = D / 32;  // output elements per lane
  constexpr int HALF = D / 2;  // elements per lane in the QK phase (two lanes per token)
  __shared__ float sq[MAXG][D];
  __shared__ float sm_m[4][MAXG], sm_l[4][MAXG];
  __shared__ float sm_o[4][MAXG][D];
  // the 16 levels, one copy per bank: lane l reads lv[code * 32 + l], so a warp never conflicts
  // (a table in constant memory would serialise the 32 different indices of a warp)
  __shared__ float lv[16 * 32];
  for (int i = threadIdx.x; i < 16 * 32; i += blockDim.x) lv[i] = c_kv_levels[i >> 5];
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = H / Hkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seq = tree.row_seq ? tree.row_seq[b] : b;
  const int len = seq_lens[seq];
  const int tail0 = tree.tail_start ? tree.tail_start[b] : len;
  const unsigned long long tail_bits = tree.tail_mask ? tree.tail_mask[b] : 0ull;
  const int npages = (len + PAGE - 1) / PAGE;
  const int per = (npages + splits - 1) / splits;
  const int p0 = split * per, p1 = min(npages, p0 + per);
  const float c = scale * 1.4426950408889634f;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, e = i % D;
    sq[g][e] = __bfloat162float(q[(long)b * ld_q + (hk * G + g) * D + e]) * c;
  }
  __syncthreads();
  float m[MAXG], l[MAXG], o[MAXG][EPL];
#pragma unroll
  for (int g = 0; g < MAXG; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[g][e] = 0.f;
  }
  const int t = lane & 15, hf = lane >> 4;
  for (int pg = p0 + warp; pg < p1; pg += 4) {
    const int page = page_table[(long)seq * max_pages + pg];
    const long row0 = ((long)page * Hkv + hk) * PAGE;
    // ---- scores: lane = (token t, half hf) ----
    float kf[HALF];
    if (OIL4) {
      const uint8_t* kp = k_pool + (row0 + t) * (D / 2) + hf * (HALF / 2);
      const __half* ks = k_scale + (row0 + t) * (D / 32) + hf * (HALF / 32);
#pragma unroll
      for (int j = 0; j < HALF / 32; ++j) {
        const float s = __half2float(ks[j]);
        const uint4 raw = *reinterpret_cast<const uint4*>(kp + j * 16);
        const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int w = 0; w < 4; ++w)
#pragma unroll
          for (int n = 0; n < 8; ++n) kf[j * 32 + w * 8 + n] = lv[(((wds[w] >> (4 * n)) & 15) << 5) + lane] * s;
      }
    } else {
      const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(k_pool) + (row0 + t) * D + hf * HALF;
#pragma unroll
      for (int j = 0; j < HALF / 8; ++j) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kp + j * 8);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const float2 f = __bfloat1622float2(h2[n]);
          kf[j * 8 + 2 * n] = f.x;
          kf[j * 8 + 2 * n + 1] = f.y;
        }
      }
    }
    const bool valid = token_visible(pg * PAGE + t, len, tail0, tail_bits);
    float pr[MAXG], alpha[MAXG];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
      if (g < G) {
        float s = 0.f;
        const float* qg = &sq[g][hf * HALF];
#pragma unroll
        for (int e = 0; e < HALF; ++e) s += kf[e] * qg[e];
        s += __shfl_xor_sync(0xffffffffu, s, 16);
        s = valid ? s : -INFINITY;
        float mx = s;
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float m_new = fmaxf(m[g], mx);
        alpha[g] = m[g] == -INFINITY ? 0.f : exp2f(m[g] - m_new);
        pr[g] = (s == -INFINITY) ? 0.f : exp2f(s - m_new);
        float ps = pr[g];
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
        l[g] = l[g] * alpha[g] + ps;
        m[g] = m_new;
      }
    }
    // ---- values: lane owns output elements [lane*EPL, lane*EPL+EPL) ----
#pragma unroll
    for (int g = 0; g < MAXG; ++g)
      if (g < G)
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[g][e] *= alpha[g];
    const int ntok = min(PAGE, len - pg * PAGE);
    for (int tt = 0; tt < ntok; ++tt) {
      float vf[EPL];
      if (OIL4) {
        const uint8_t* vp = v_pool + (row0 + tt) * (D / 2) + (lane * EPL) / 2;
        const float s = __half2float(v_scale[(row0 + tt) * (D / 32) + (lane * EPL) / 32]);
        uint32_t bits = EPL == 4 ? *reinterpret_cast<const uint16_t*>(vp) : *vp;
#pragma unroll
        for (int e = 0; e < EPL; ++e) vf[e] = lv[(((bits >> (4 * e)) & 15) << 5) + lane] * s;
      } else {
        const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(v_pool) + (row0 + tt) * D + lane * EPL;
#pragma unroll
        for (int e = 0; e < EPL; ++e) vf[e] = __bfloat162float(vp[e]);
      }
#pragma unroll
      for (int g = 0; g < MAXG; ++g)
        if (g < G) {
          const float pt = __shfl_sync(0xffffffffu, pr[g], tt);
#pragma unroll
          for (int e = 0; e < EPL; ++e) o[g][e] += pt * vf[e];
        }
    }
  }
  // ---- fold the 4 warps ----
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      sm_m[warp][g] = m[g];
      sm_l[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_o[warp][g][lane * EPL + e] = o[g][e];
  }
  __syncthreads();
  float* out = part + (((long)b * Hkv + hk) * splits + split) * (long)G * (D + 2);
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, e = i % D;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float acc = 0.f, ll = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float f = sm_m[w][g] == -INFINITY ? 0.f : exp2f(sm_m[w][g] - mm);
      acc += sm_o[w][g][e] * f;
      ll += sm_l[w][g] * f;
    }
    out[g * (D + 2) + 2 + e] = acc;
    if (e == 0) {
      out[g * (D + 2)] = mm;
      out[g * (D + 2) + 1] = ll;
    }
  }
}

// OIL4 decode attention on the tensor cores (warp-level mma.sync m16n8k16, fp16 inputs, fp32 accumulation).
// A GQA group has at most 8 query heads per KV head, far below the 64-row minimum of tcgen05.mma, and the kernel
// is bound by index bytes and table lookups, not by tensor throughput, so the warp-level MMA is the right size:
// one warp owns one 16-token page at a time and never touches shared memory except for the lookup table.
//   scores  S[head, token]  = Q[head, d] . K[token, d]^T   A = Q (rows >= G are zero), B = K: lane (token = lane/4,
//           quarter = lane%4) expands the 16 index bytes of its token's d-quarter; since the contraction runs over
//           d, the d order inside the MMA is permuted so that every lane feeds its own bytes in order
//   softmax on the accumulator fragment (lane holds 4 tokens of head lane/4), running max / sum per head
//   values  O^T[d, head]    = V^T[d, token] . P^T[token, head]   B = P^T is the score fragment as it stands, A = V^T:
//           lane (d-chunk = lane/4) expands 8 bytes of four tokens and pairs values of neighbouring tokens with
//           byte permutes; the output d order is permuted the same way and undone when the result is written
// K, V and their scales for the next page are loaded before the current page is processed.
__device__ __forceinline__ void mma_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

template <int D, int NW>
__global__ void __launch_bounds__(NW * 32, 512 / (NW * 32)) paged_decode_oil4_mma_kernel(const __nv_bfloat16* __restrict__ q, int ld_q, const int* __restrict__ page_table,
                                                                    int max_pages, const int* __restrict__ seq_lens, int H, int Hkv,
                                                                    const uint8_t* __restrict__ k_pool, const uint8_t* __restrict__ v_pool,
                                                                    const __half* __restrict__ k_scale, const __half* __restrict__ v_scale,
                                                                    float scale, float* __restrict__ part, int splits,
                                                                    __nv_bfloat16* __restrict__ out_direct, int ld_o, TreeRows tree) {
  constexpr int MAXG = 8;
  constexpr int KCH = D / 4;        // d-values of a K row per lane (one quarter of the row)
  constexpr int KW = KCH / 8;       // ... as 32-bit words of indices (4 for D = 128)
  constexpr int KSTEPS = KCH / 4;   // MMA k-steps: 4 d-values per lane and step
  constexpr int VCH = D / 8;        // d-values of a V row per lane (one eighth of the row)
  constexpr int VW = VCH / 8;       // ... as 32-bit words (2 for D = 128)
  constexpr int VMMA = VCH / 2;     // PV MMAs per page: 2 d-values per lane and MMA
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the output projection may start on its weights
  __shared__ __align__(16) uint32_t lut[256 * 32];  // byte -> half2(level[low nibble], level[high nibble]); entry e of lane l at [e * 32 + l]
  __shared__ float sm_m[NW][MAXG], sm_l[NW][MAXG];
  float (*sm_o)[MAXG][D] = reinterpret_cast<float (*)[MAXG][D]>(lut);  // the per-warp outputs reuse the table once the loop is over
  for (int i4 = threadIdx.x; i4 < 256 * 8; i4 += blockDim.x) {
    const int e = i4 >> 3;
    const uint32_t v = h2_as_u32(__floats2half2_rn(c_kv_levels[e & 15], c_kv_levels[e >> 4]));
    *reinterpret_cast<uint4*>(&lut[i4 * 4]) = make_uint4(v, v, v, v);
  }
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = H / Hkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int seq = tree.row_seq ? tree.row_seq[b] : b;
  const int len = seq_lens[seq];
  const int tail0 = tree.tail_start ? tree.tail_start[b] : len;
  const unsigned long long tail_bits = tree.tail_mask ? tree.tail_mask[b] : 0ull;
  const int npages = (len + PAGE - 1) / PAGE;
  const int per = (npages + splits - 1) / splits;
  const int p0 = split * per, p1 = min(npages, p0 + per);
  const float c = scale * 1.4426950408889634f;
  // Q fragment: row gid = query head, this lane's d-quarter; rows 8..15 of the MMA are zero
  uint32_t qa[KSTEPS][2];
  {
    const __nv_bfloat16* qrow = q + (long)b * ld_q + (hk * G + min(gid, G - 1)) * D + tig * KCH;
#pragma unroll
    for (int st = 0; st < KSTEPS; ++st) {
      const uint2 raw = *reinterpret_cast<const uint2*>(qrow + st * 4);
      const float f0 = __uint_as_float(raw.x << 16) * c, f1 = __uint_as_float(raw.x & 0xffff0000u) * c;
      const float f2 = __uint_as_float(raw.y << 16) * c, f3 = __uint_as_float(raw.y & 0xffff0000u) * c;
      qa[st][0] = gid < G ? h2_as_u32(__floats2half2_rn(f0, f1)) : 0u;
      qa[st][1] = gid < G ? h2_as_u32(__floats2half2_rn(f2, f3)) : 0u;
    }
  }
  __syncthreads();
  float m_run = -INFINITY, l_run = 0.f;  // of head gid; l is this lane's share (its 4 tokens per page)
  float o[VMMA][4];
#pragma unroll
  for (int i = 0; i < VMMA; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  uint32_t kraw[2][KW], vraw[4][VW];
  __half ksc[2], vsc[4];
  auto fetch = [&](int pg) {
    const int page = page_table[(long)seq * max_pages + pg];
    const long row0 = ((long)page * Hkv + hk) * PAGE;
#pragma unroll
    for (int t = 0; t < 2; ++t) {  // K: tokens gid and gid + 8, bytes of d-quarter tig
      const long row = row0 + gid + 8 * t;
      const uint8_t* kp = k_pool + row * (D / 2) + tig * (KCH / 2);
      if (KW == 4) {
        const uint4 v4 = *reinterpret_cast<const uint4*>(kp);
        kraw[t][0] = v4.x; kraw[t][1] = v4.y; kraw[t][2 % KW] = v4.z; kraw[t][3 % KW] = v4.w;
      } else {
        const uint2 v2 = *reinterpret_cast<const uint2*>(kp);
        kraw[t][0] = v2.x; kraw[t][1] = v2.y;
      }
      ksc[t] = k_scale[row * (D / 32) + (tig * KCH) / 32];
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {  // V: tokens 2 tig, 2 tig + 1, 2 tig + 8, 2 tig + 9, bytes of d-chunk gid
      const long row = row0 + 2 * tig + (t & 1) + 8 * (t >> 1);
      const uint8_t* vp = v_pool + row * (D / 2) + gid * (VCH / 2);
      if (VW == 2) {
        const uint2 v2 = *reinterpret_cast<const uint2*>(vp);
        vraw[t][0] = v2.x; vraw[t][1 % VW] = v2.y;
      } else {
        vraw[t][0] = *reinterpret_cast<const uint32_t*>(vp);
      }
      vsc[t] = v_scale[row * (D / 32) + (gid * VCH) / 32];
    }
  };
  int pg = p0 + warp;
  if (pg < p1) fetch(pg);
  for (; pg < p1; pg += NW) {
    // ---- this page's registers; then start the next page's loads ----
    uint32_t kr[2][KW], vr[4][VW];
    __half2 ks2[2], vs2[4];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
#pragma unroll
      for (int w = 0; w < KW; ++w) kr[t][w] = kraw[t][w];
      ks2[t] = __half2half2(ksc[t]);
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
#pragma unroll
      for (int w = 0; w < VW; ++w) vr[t][w] = vraw[t][w];
      const int tok = pg * PAGE + 2 * tig + (t & 1) + 8 * (t >> 1);
      vs2[t] = tok < len ? __half2half2(vsc[t]) : __float2half2_rn(0.f);  // rows past the end may hold anything
    }
    if (pg + NW < p1) fetch(pg + NW);
    // ---- scores: two n-tiles of 8 tokens ----
    float s[2][4];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
#pragma unroll
      for (int st = 0; st < KSTEPS; ++st) {
        // bytes 2 st and 2 st + 1 of the lane's chunk: d-values 4 st .. 4 st + 3
        const uint32_t two = kr[t][st >> 1] >> (16 * (st & 1));
        const __half2 k01 = __hmul2(u32_as_h2(lut[((two & 255) << 5) + lane]), ks2[t]);
        const __half2 k23 = __hmul2(u32_as_h2(lut[(((two >> 8) & 255) << 5) + lane]), ks2[t]);
        const uint32_t a[4] = {qa[st][0], 0u, qa[st][1], 0u};
        mma_16816(s[t], a, h2_as_u32(k01), h2_as_u32(k23));
      }
    }
    // lane: head gid, tokens {2 tig, 2 tig + 1} (+ 8 for the second tile) in s[t][0], s[t][1]
    float sv[4];
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = pg * PAGE + 8 * t + 2 * tig + e;
        sv[t * 2 + e] = token_visible(tok, len, tail0, tail_bits) ? s[t][e] : -INFINITY;
      }
    float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    // -inf only while a tree row has met nothing but other branches' tokens: keep the exponent arguments defined
    const float m_ref = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = exp2f(m_run - m_ref);  // 0 on the first page (m_run = -inf)
    float pe[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pe[i] = exp2f(sv[i] - m_ref);
    l_run = l_run * alpha + (pe[0] + pe[1]) + (pe[2] + pe[3]);
    m_run = m_new;
    const uint32_t pb0 = h2_as_u32(__floats2half2_rn(pe[0], pe[1])), pb1 = h2_as_u32(__floats2half2_rn(pe[2], pe[3]));
    // ---- rescale O^T: this lane's columns are heads 2 tig and 2 tig + 1, whose factors live in lanes 8 tig, 8 tig + 4 ----
    const float al0 = __shfl_sync(0xffffffffu, alpha, 8 * tig), al1 = __shfl_sync(0xffffffffu, alpha, 8 * tig + 4);
    if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
      for (int i = 0; i < VMMA; ++i) {
        o[i][0] *= al0; o[i][1] *= al1; o[i][2] *= al0; o[i][3] *= al1;
      }
    }
    // ---- values: MMA i covers d = gid * VCH + 2 i (row gid) and + 1 (row gid + 8) ----
#pragma unroll
    for (int i = 0; i < VMMA; ++i) {
      __half2 x[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t byte = (vr[t][i >> 2] >> (8 * (i & 3))) & 255;
        x[t] = __hmul2(u32_as_h2(lut[(byte << 5) + lane]), vs2[t]);  // (V[token t][d], V[token t][d + 1])
      }
      uint32_t a[4];
      a[0] = __byte_perm(h2_as_u32(x[0]), h2_as_u32(x[1]), 0x5410);  // row d,     tokens 2 tig, 2 tig + 1
      a[1] = __byte_perm(h2_as_u32(x[0]), h2_as_u32(x[1]), 0x7632);  // row d + 1, same tokens
      a[2] = __byte_perm(h2_as_u32(x[2]), h2_as_u32(x[3]), 0x5410);  // row d,     tokens + 8
      a[3] = __byte_perm(h2_as_u32(x[2]), h2_as_u32(x[3]), 0x7632);
      mma_16816(o[i], a, pb0, pb1);
    }
  }
  // ---- fold the lanes' shares of l, then the 4 warps ----
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (tig == 0 && gid < G) {
    sm_m[warp][gid] = m_run;
    sm_l[warp][gid] = l_run;
  }
  __syncthreads();  // every warp is done with the table
#pragma unroll
  for (int i = 0; i < VMMA; ++i) {
    const int d0 = gid * VCH + 2 * i;
    if (2 * tig < G) {
      sm_o[warp][2 * tig][d0] = o[i][0];
      sm_o[warp][2 * tig][d0 + 1] = o[i][2];
    }
    if (2 * tig + 1 < G) {
      sm_o[warp][2 * tig + 1][d0] = o[i][1];
      sm_o[warp][2 * tig + 1][d0 + 1] = o[i][3];
    }
  }
  __syncthreads();
  float* out = part + (((long)b * Hkv + hk) * splits + split) * (long)G * (D + 2);
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, e = i % D;
    float mm = -INFINITY;
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float acc = 0.f, ll = 0.f;
    for (int w = 0; w < NW; ++w) {
      const float f = sm_m[w][g] == -INFINITY ? 0.f : exp2f(sm_m[w][g] - mm);
      acc += sm_o[w][g][e] * f;
      ll += sm_l[w][g] * f;
    }
    if (out_direct != nullptr) {  // a single split: the result is final, no combine pass
      out_direct[(long)b * ld_o + (hk * G + g) * D + e] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
      continue;
    }
    out[g * (D + 2) + 2 + e] = acc;
    if (e == 0) {
      out[g * (D + 2)] = mm;
      out[g * (D + 2) + 1] = ll;
    }
  }
}

// out[b, h*D + e] = sum_s o_s * 2^(m_s - m) / sum_s l_s * 2^(m_s - m)
__global__ void attn_combine_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int ld_o, int B, int H, int Hkv, int D,
                                    int splits) {
  const int G = H / Hkv;
  const long total = (long)B * H * D;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int e = (int)(i % D);
    const int h = (int)((i / D) % H);
    const int b = (int)(i / ((long)D * H));
    const int hk = h / G, g = h % G;
    const float* base = part + (((long)b * Hkv + hk) * splits) * (long)G * (D + 2) + g * (D + 2);
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, base[(long)s * G * (D + 2)]);
    float acc = 0.f, ll = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* ps = base + (long)s * G * (D + 2);
      const float f = ps[0] == -INFINITY ? 0.f : exp2f(ps[0] - mm);
      acc += ps[2 + e] * f;
      ll += ps[1] * f;
    }
    out[(long)b * ld_o + h * D + e] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
  }
}

}  // namespace inv

using namespace inv;

extern "C" int inv_kv_append(const void* k_new, const void* v_new, int ld_k, int ld_v, const int* page_table, int max_pages, const int* start_pos,
                             int B, int S_new, int Hkv, int D, void* k_pool, void* v_pool, void* k_scale, void* v_scale, int oil4,
                             void* stream) {
  if (D % 32 || B <= 0 || S_new <= 0) return B <= 0 || S_new <= 0 ? 0 : -ERR_BAD_ARG;
  const long warps = (long)B * S_new * Hkv * 2;
  const int grid = (int)((warps + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (oil4)
    kv_append_kernel<true><<<grid, 256, 0, st>>>((const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, ld_k, ld_v, page_table, max_pages,
                                                 start_pos, B, S_new, Hkv, D, (uint8_t*)k_pool, (uint8_t*)v_pool, (__half*)k_scale,
                                                 (__half*)v_scale);
  else
    kv_append_kernel<false><<<grid, 256, 0, st>>>((const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, ld_k, ld_v, page_table, max_pages,
                                                  start_pos, B, S_new, Hkv, D, (uint8_t*)k_pool, (uint8_t*)v_pool, (__half*)k_scale,
                                                  (__half*)v_scale);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

namespace inv {
// Decode-step finish of the QKV projection: one pass over the fp32 accumulator [B, (H + 2 Hkv) D] that adds the bias,
// rounds to bf16 (as the stand-alone finish pass does), rotates the query and key heads (half-split RoPE at the token's
// position), writes the queries as bf16 and appends the key / value heads to the paged cache (OIL4: block-32 abs-max
// scale + nearest of the 16 levels; or bf16), and clears the accumulator. Replaces three launches per layer.
// One warp per (token, head slot); lane l owns elements l + 32 j, so a rotation pair (e, e + D/2) sits in one thread.
template <bool OIL4, int D>
__global__ void __launch_bounds__(256) decode_qkv_finish_kernel(float* __restrict__ acc, int ld_acc, const __nv_bfloat16* __restrict__ bias,
                                                                const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                                const int* __restrict__ pos, const int* __restrict__ page_table, int max_pages,
                                                                int B, int H, int Hkv, __nv_bfloat16* __restrict__ q_out, int ld_q,
                                                                uint8_t* __restrict__ k_pool, uint8_t* __restrict__ v_pool,
                                                                __half* __restrict__ k_scale, __half* __restrict__ v_scale) {
  constexpr int NJ = D / 32, HALFJ = NJ / 2;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const long warp_id = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int slots = H + 2 * Hkv;
  if (warp_id >= (long)B * slots) return;
  const int slot = (int)(warp_id % slots), b = (int)(warp_id / slots);
  float* arow = acc + (size_t)b * ld_acc + slot * D;
  float v[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int e = lane + 32 * j;
    float x = arow[e];
    arow[e] = 0.f;
    if (bias) x += __bfloat162float(bias[slot * D + e]);
    v[j] = __bfloat162float(__float2bfloat16_rn(x));
  }
  const int p = pos[b];
  if (slot < H + Hkv) {  // query and key heads rotate
#pragma unroll
    for (int j = 0; j < HALFJ; ++j) {
      const int i = lane + 32 * j;
      const float c = cos_t[(size_t)p * (D / 2) + i], sn = sin_t[(size_t)p * (D / 2) + i];
      const float x1 = v[j], x2 = v[j + HALFJ];
      v[j] = __bfloat162float(__float2bfloat16_rn(x1 * c - x2 * sn));
      v[j + HALFJ] = __bfloat162float(__float2bfloat16_rn(x1 * sn + x2 * c));
    }
  }
  if (slot < H) {
    __nv_bfloat16* qo = q_out + (size_t)b * ld_q + slot * D;
#pragma unroll
    for (int j = 0; j < NJ; ++j) qo[lane + 32 * j] = __float2bfloat16_rn(v[j]);
    return;
  }
  const int which = slot >= H + Hkv;  // 0 = key, 1 = value
  const int hk = slot - H - which * Hkv;
  const int page = page_table[(long)b * max_pages + p / PAGE];
  const long row = ((long)page * Hkv + hk) * PAGE + p % PAGE;
  uint8_t* pool = which ? v_pool : k_pool;
  if (!OIL4) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(pool) + row * D;
#pragma unroll
    for (int j = 0; j < NJ; ++j) dst[lane + 32 * j] = __float2bfloat16_rn(v[j]);
    return;
  }
  __half* sc = (which ? v_scale : k_scale) + row * (D / 32);
  uint8_t* dst = pool + row * (D / 2);
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    float amax = fabsf(v[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax < 1e-10f ? 1.f : amax;
    const int code = nearest_level16(v[j] / scale);
    const int hi = __shfl_down_sync(0xffffffffu, code, 1);
    if ((lane & 1) == 0) dst[j * 16 + (lane >> 1)] = (uint8_t)(code | (hi << 4));
    if (lane == 0) sc[j] = __float2half_rn(scale);
  }
}

}  // namespace inv
using namespace inv;
extern "C" int inv_decode_qkv_finish(float* acc, int ld_acc, const void* bias, const float* cos_t, const float* sin_t, const int* pos,
                                     const int* page_table, int max_pages, int B, int H, int Hkv, int D, void* q_out, int ld_q, void* k_pool,
                                     void* v_pool, void* k_scale, void* v_scale, int oil4, void* stream) {
  if (D != 64 && D != 128) return -ERR_BAD_ARG;
  if (B <= 0) return 0;
  const long warps = (long)B * (H + 2 * Hkv);
  const int grid = (int)((warps + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
#define INV_DQF(O, DD)                                                                                                                      \
  decode_qkv_finish_kernel<O, DD><<<grid, 256, 0, st>>>(acc, ld_acc, (const __nv_bfloat16*)bias, cos_t, sin_t, pos, page_table, max_pages, B, \
                                                        H, Hkv, (__nv_bfloat16*)q_out, ld_q, (uint8_t*)k_pool, (uint8_t*)v_pool,             \
                                                        (__half*)k_scale, (__half*)v_scale)
  if (oil4) {
    if (D == 64) INV_DQF(true, 64); else INV_DQF(true, 128);
  } else {
    if (D == 64) INV_DQF(false, 64); else INV_DQF(false, 128);
  }
#undef INV_DQF
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// Scratch floats needed by inv_paged_decode.
extern "C" long inv_paged_decode_scratch_floats(int B, int H, int D, int splits) { return (long)B * H * splits * (D + 2); }

static int paged_decode_impl(const void* q, int ld_q, const int* page_table, int max_pages, const int* seq_lens, int B, int H, int Hkv, int D,
                             const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale, int oil4, float scale,
                             void* out, int ld_o, float* scratch, int splits, TreeRows tree, void* stream) {
  if ((D != 64 && D != 128) || H % Hkv || H / Hkv > 8 || splits < 1) return -ERR_BAD_ARG;
  if (B <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(splits, Hkv, B);
#define INV_PD(O, DD)                                                                                                                      \
  paged_decode_kernel<O, DD><<<grid, 128, 0, st>>>((const __nv_bfloat16*)q, ld_q, page_table, max_pages, seq_lens, H, Hkv,                 \
                                                   (const uint8_t*)k_pool, (const uint8_t*)v_pool, (const __half*)k_scale,                 \
                                                   (const __half*)v_scale, scale, scratch, splits, tree)
  if (oil4) {
    // four warps per CTA, four CTAs per SM. Eight warps (NW = 8, two CTAs per SM) halve a CTA's serial chain of pages but
    // double the waves of the grid: 35.7 us either way at batch 64, 8 KV heads, 640 tokens of context
#define INV_PD4(DD, NW)                                                                                                                    \
  paged_decode_oil4_mma_kernel<DD, NW><<<grid, NW * 32, 0, st>>>((const __nv_bfloat16*)q, ld_q, page_table, max_pages, seq_lens, H, Hkv,      \
                                                             (const uint8_t*)k_pool, (const uint8_t*)v_pool, (const __half*)k_scale,       \
                                                             (const __half*)v_scale, scale, scratch, splits,                                \
                                                             splits == 1 ? (__nv_bfloat16*)out : nullptr, ld_o, tree)
    if (D == 64) INV_PD4(64, 4); else INV_PD4(128, 4);
#undef INV_PD4
    if (splits == 1) {  // the kernel wrote the final output
      cudaError_t e1 = cudaGetLastError();
      return e1 == cudaSuccess ? 0 : -(int)e1;
    }
  } else {
    if (D == 64) INV_PD(false, 64); else INV_PD(false, 128);
  }
#undef INV_PD
  const long n = (long)B * H * D;
  long g = (n + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  attn_combine_kernel<<<(int)g, 256, 0, st>>>(scratch, (__nv_bfloat16*)out, ld_o, B, H, Hkv, D, splits);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_paged_decode(const void* q, int ld_q, const int* page_table, int max_pages, const int* seq_lens, int B, int H, int Hkv, int D,
                                const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale, int oil4, float scale,
                                void* out, int ld_o, float* scratch, int splits, void* stream) {
  return paged_decode_impl(q, ld_q, page_table, max_pages, seq_lens, B, H, Hkv, D, k_pool, v_pool, k_scale, v_scale, oil4, scale, out, ld_o,
                           scratch, splits, TreeRows{nullptr, nullptr, nullptr}, stream);
}

// Attention of T query rows over shared sequences with a per-row visibility mask over the newest (at most 64) tokens:
// the verification pass of tree-structured speculative decoding in one launch (include/oil/inference_opt.h:262-298).
// Row t attends sequence row_seq[t]: every cached token below tail_start[t], and token tail_start[t] + i iff bit i of
// tail_mask[t] is set. seq_lens[row_seq[t]] - tail_start[t] must not exceed 64.
extern "C" int inv_paged_decode_tree(const void* q, int ld_q, const int* page_table, int max_pages, const int* seq_lens, const int* row_seq,
                                     const int* tail_start, const unsigned long long* tail_mask, int T, int H, int Hkv, int D,
                                     const void* k_pool, const void* v_pool, const void* k_scale, const void* v_scale, int oil4, float scale,
                                     void* out, int ld_o, float* scratch, int splits, void* stream) {
  if (row_seq == nullptr || tail_start == nullptr || tail_mask == nullptr) return -ERR_BAD_ARG;
  return paged_decode_impl(q, ld_q, page_table, max_pages, seq_lens, T, H, Hkv, D, k_pool, v_pool, k_scale, v_scale, oil4, scale, out, ld_o,
                           scratch, splits, TreeRows{row_seq, tail_start, tail_mask}, stream);
}
