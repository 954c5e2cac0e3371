// Flash attention forward on tcgen05 tensor cores (causal or full, MHA or GQA, head_dim 64 or 128).
//
// Replaces the reference's flash_attention_forward (src/flash_attention.cpp:38-191: tiled online
// softmax), the autograd attention op (include/oil/autograd_functions.h:82-94) and the two-pass
// shader attention (src/gpu_compute_full.cpp:306-348).
//
// Layout: q, k, v are token-major views [B*S, ld] of one fused qkv buffer; head h of q occupies
// columns [h*D, (h+1)*D). The output is token-major [B*S, H*D], ready for the o-projection GEMM.
//
// One CTA per (batch, head, 128-query block), 192 threads:
//   warp 0    TMA producer: Q once, then K_j / V_j tiles through a ring of five (D = 64) or four slots (128B swizzle).
//   warp 1    MMA issuer: S = Q K_j^T (128x128 fp32 in TMEM), then O += P_j V_j (128xD in TMEM, P read from TMEM).
//   warps 2-5 softmax, one query row per thread: read S from TMEM, online max / exp2 / sum, write P_j back to
//             tensor memory as packed bf16 (the A operand of the PV MMA); O and the row sums stay in TMEM with a lazy rescale.
// For D = 64 two CTAs share an SM, so one CTA's softmax overlaps the other's MMAs. Every wait is bounded and
// reports through *status.
#include "sm100_common.cuh"
#include "inv_api.h"

#include <mutex>

namespace inv {

constexpr int FA_BM = 128, FA_BN = 128;
constexpr int FA_THREADS = 192;

struct FlashFwdParams {
  __nv_bfloat16* out;
  int ld_o;
  float* lse;  // [B, H, S], log2 of the softmax denominator (scores scaled by scale*log2 e)
  int B, S, H, Hkv;
  float scale;
  int causal;
  int window;  // > 0 (causal only): a query sees the `window` most recent keys, its own position included
  int* status;
};

// ------------------------------------------------------------------------------------------------
// Forward kernel. Cycle stamps of an earlier layout (P staged through shared memory, three K/V ring slots)
// showed where a key block's ~4000 cycles went: ~1500 waiting for a K tile (the load of K_{j+1} could
// not start before P_{j-1}V_{j-1} had finished), ~1000 waiting for the previous PV MMA before the
// exponentials even started, ~1200 in the PV MMA plus a separate row-sum MMA, and ~1800 in the
// exponential phase itself (MUFU-bound). This kernel
//   * keeps P in tensor memory: the softmax threads write packed bf16 pairs with tcgen05.st and the PV MMA
//     reads its A operand from TMEM, so the 32 KB shared-memory P tile, its stores and the proxy fence are
//     gone and the K/V ring grows to five slots (loads run two key blocks ahead);
//   * computes the exponentials into registers *before* it waits for the previous PV MMA, which is only
//     needed for the TMEM store of P (and the rare rescale of O);
//   * sums the exponentials on the FMA pipe: packed bf16 adds over groups of four, then fp32.
// TMEM columns per CTA: S [0,128) fp32, O [128,128+D) fp32, P [128+D, 192+D) packed bf16.
// ------------------------------------------------------------------------------------------------
template <int ND>
struct Fwd3Smem {
  static constexpr int TILE = ND * 16384;
  static constexpr int SLOTS = ND == 1 ? 5 : 4;
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = TILE;
  static constexpr int BAR_OFF = KV_OFF + SLOTS * TILE;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int ND>
__global__ void __launch_bounds__(FA_THREADS, ND == 1 ? 2 : 1)
flash_fwd3_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const FlashFwdParams p) {
  constexpr int D = 64 * ND;
  using L = Fwd3Smem<ND>;
  constexpr int SLOTS = L::SLOTS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sKV = smem + L::KV_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;              // 1
  uint64_t* kv_full = bars + 1;         // SLOTS
  uint64_t* kv_empty = bars + 1 + SLOTS;  // SLOTS
  uint64_t* s_full = bars + 1 + 2 * SLOTS;
  uint64_t* s_empty = s_full + 1;       // 128 arrivals
  uint64_t* p_full = s_full + 2;        // 128 arrivals
  uint64_t* o_full = s_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + FA_BM - 1) / FA_BM;
  const int q_blk = nqb - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = q_blk * FA_BM;
  const int nkb_all = (p.S + FA_BN - 1) / FA_BN;
  // key blocks visited: [jlo, jlo + nkb). A sliding window skips the blocks that lie wholly before the first query's window.
  const int jlo = (p.causal && p.window > 0) ? max(0, q0 - p.window + 1) / FA_BN : 0;
  const int nkb = (p.causal ? min(nkb_all, q_blk + 1) : nkb_all) - jlo;
  constexpr uint32_t TMEM_COLS = ND == 1 ? 256 : 512;
  constexpr uint32_t O_COL = 128, P_COL = 128 + D;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < SLOTS; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 4);
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, L::TILE);
#pragma unroll
      for (int a = 0; a < ND; ++a) tma_load_3d(sQ + a * 16384, &tmap_q, q_full, h * D + a * 64, q0, b);
      for (int n = 0; n < 2 * nkb; ++n) {
        const int slot = n % SLOTS;
        const uint32_t ph = (n / SLOTS) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&kv_full[slot], L::TILE);
        const int j = jlo + (n >> 1);
        const CUtensorMap* tm = (n & 1) ? &tmap_v : &tmap_k;
#pragma unroll
        for (int a = 0; a < ND; ++a) tma_load_3d(sKV + slot * L::TILE + a * 16384, tm, &kv_full[slot], hk * D + a * 64, j * FA_BN, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);
      const uint32_t q_base = smem_u32(sQ);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ERR_WAIT_FULL);
      auto issue_qk = [&](int j) -> bool {
        const int n = 2 * j, slot = n % SLOTS;
        if (!mbar_wait(&kv_full[slot], (n / SLOTS) & 1, abort_flag, p.status, ERR_WAIT_FULL)) return false;
        if (j > 0 && !mbar_wait(s_empty, (j - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t k_base = smem_u32(sKV + slot * L::TILE);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
          umma_bf16(tmem_base, make_smem_desc(q_base + off, 16, 1024, 2), make_smem_desc(k_base + off, 16, 1024, 2), idesc_qk, ks > 0);
        }
        umma_commit(s_full);
        umma_commit(&kv_empty[slot]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < nkb; ++j) {
        if (j + 1 < nkb) {
          if (!issue_qk(j + 1)) break;
        }
        const int n = 2 * j + 1, slot = n % SLOTS;
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status, ERR_WAIT_MISC)) break;
        if (!mbar_wait(&kv_full[slot], (n / SLOTS) & 1, abort_flag, p.status, ERR_WAIT_FULL)) break;
        tc_fence_after();
        const uint32_t v_base = smem_u32(sKV + slot * L::TILE);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks)  // 16 keys = 8 packed columns of P per step
          umma_bf16_tmem_a(tmem_base + O_COL, tmem_base + P_COL + ks * 8, make_smem_desc(v_base + ks * 2048, 16384, 1024, 2), idesc_pv,
                           (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(&kv_empty[slot]);
      }
    }
  } else {
    // ---------------- softmax warps: thread <-> query row ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int row = q0 + r;
    const uint32_t t_lane = tmem_base + (uint32_t(q * 32) << 16);
    const float c = p.scale * 1.4426950408889634f;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkb; ++j) {
      if (!mbar_wait_warp(s_full, j & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = (jlo + j) * FA_BN;
      const bool windowed = p.causal && p.window > 0;
      const bool need_mask = (p.causal && k0 + FA_BN - 1 > q0) || (k0 + FA_BN > p.S) || (windowed && k0 <= q0 + FA_BM - 1 - p.window);
      const int kmax = p.causal ? min(row, p.S - 1) : p.S - 1;
      const int kmin = windowed ? row - p.window + 1 : 0;
      uint32_t sr[128];
      tmem_ld_32x32(t_lane, sr);
      tmem_ld_32x32(t_lane + 32, sr + 32);
      tmem_ld_32x32(t_lane + 64, sr + 64);
      tmem_ld_32x32(t_lane + 96, sr + 96);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);  // the scores live in registers now: the next QK^T may start (one arrival per warp)
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (k0 + i > kmax || k0 + i < kmin) sr[i] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 8) {
        mx0 = fmax3(mx0, __uint_as_float(sr[i + 0]), __uint_as_float(sr[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
        mx2 = fmax3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
        mx3 = fmax3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
      }
      const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const bool raise = j == 0 || (m_blk - m_used) * c > 8.0f;  // lazy: tolerate exponents up to 2^8
      const float m_new = raise ? fmaxf(m_used, m_blk) : m_used;
      const float alpha = (j == 0 || !raise) ? 1.0f : exp2f((m_used - m_new) * c);
      m_used = m_new;
      const bool any_rescale = __any_sync(0xffffffffu, j > 0 && raise);
      const float mc = m_used == -INFINITY ? 0.f : m_used * c;  // a row that has seen no key yet (window edge): every exponential is 0
      // exponentials into registers (packed bf16 pairs overwrite the scores) and their sum: one MUFU op per element and
      // one hardware conversion per pair
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int i = 0; i < 128; i += 2) {
        const float e0 = exp2f(fmaf(__uint_as_float(sr[i]), c, -mc));
        const float e1 = exp2f(fmaf(__uint_as_float(sr[i + 1]), c, -mc));
        rs0 += e0;
        rs1 += e1;
        sr[i >> 1] = cvt_bf16x2(e0, e1);  // slot i/2 <= i: never read again as a score
      }
      l = l * alpha + (rs0 + rs1);
      if (j > 0) {
        // PV of the previous block is complete: P may be overwritten, O is stable
        if (!mbar_wait_warp(o_full, (j - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        if (any_rescale) {
#pragma unroll 1
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t rr[32];
            tmem_ld_32x32(t_lane + O_COL + cc * 32, rr);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * alpha);
            tmem_st_32x32(t_lane + O_COL + cc * 32, rr);
          }
        }
      }
      tmem_st_32x32(t_lane + P_COL, sr);
      tmem_st_32x32(t_lane + P_COL + 32, sr + 32);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) ok = mbar_wait_warp(o_full, (nkb - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)b * p.S + row) * p.ld_o + h * D;
#pragma unroll 1
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t rr[32];
        tmem_ld_32x32(t_lane + O_COL + cc * 32, rr);
        tmem_ld_wait();
        if (row < p.S) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(rr[g * 8 + 0]) * inv_l, __uint_as_float(rr[g * 8 + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(rr[g * 8 + 2]) * inv_l, __uint_as_float(rr[g * 8 + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(rr[g * 8 + 4]) * inv_l, __uint_as_float(rr[g * 8 + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(rr[g * 8 + 6]) * inv_l, __uint_as_float(rr[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(dst + cc * 32 + g * 8) = o;
          }
        }
      }
      if (p.lse && row < p.S) p.lse[((size_t)b * p.H + h) * p.S + row] = m_used * c + log2f(l);
      tc_fence_before();
    }
  }

  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// 3-D bf16 tensor map over a token-major buffer: dims {cols, S, B}, box {64, rows, 1}, 128B swizzle.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn fa_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}
int make_tmap_tokens_bf16(CUtensorMap* out, const void* ptr, int cols, int S, int B, int ld, int box_rows) {
  EncodeTiledFn enc = fa_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)S * ld * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

// fp32 [B, S, cols] (dense rows): boxes of 32 rows x 16 floats, 64-byte swizzle.
int make_tmap_tokens_f32(CUtensorMap* out, const void* ptr, int cols, int S, int B) {
  EncodeTiledFn enc = fa_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 4, (cuuint64_t)S * cols * 4};
  cuuint32_t box[3] = {16, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

}  // namespace inv

using namespace inv;

// q/k/v: token-major bf16 [B*S, ld*]; q has H heads, k and v have Hkv heads of `head_dim` columns.
// out: [B*S, ld_o] bf16; lse: [B, H, S] fp32 (may be null).
extern "C" int inv_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int H, int Hkv,
                                  int head_dim, int ld_q, int ld_k, int ld_v, int ld_o, float scale, int causal, int window, int* status,
                                  void* stream) {
  if ((head_dim != 64 && head_dim != 128) || H % Hkv || (ld_q % 8) || (ld_k % 8) || (ld_v % 8) || (ld_o % 8)) return -ERR_BAD_ARG;
  if (window < 0 || (window > 0 && !causal)) return -ERR_BAD_ARG;  // the sliding window is defined for causal attention
  if (B <= 0 || S <= 0) return 0;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_tokens_bf16(&tq, q, H * head_dim, S, B, ld_q, FA_BM))) return rc;
  if ((rc = make_tmap_tokens_bf16(&tk, k, Hkv * head_dim, S, B, ld_k, FA_BN))) return rc;
  if ((rc = make_tmap_tokens_bf16(&tv, v, Hkv * head_dim, S, B, ld_v, FA_BN))) return rc;
  FlashFwdParams p;
  p.out = (__nv_bfloat16*)out; p.ld_o = ld_o; p.lse = lse;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv; p.scale = scale; p.causal = causal; p.window = 0; p.status = status;
  dim3 grid((S + FA_BM - 1) / FA_BM, H, B);
  cudaStream_t st = (cudaStream_t)stream;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(flash_fwd3_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd3Smem<1>::TOTAL);
    cudaFuncSetAttribute(flash_fwd3_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd3Smem<2>::TOTAL);
    configured = true;
  }
  p.causal = causal ? 1 : 0;
  p.window = window >= S ? 0 : window;
  if (head_dim == 64) flash_fwd3_kernel<1><<<grid, FA_THREADS, Fwd3Smem<1>::TOTAL, st>>>(tq, tk, tv, p);
  else flash_fwd3_kernel<2><<<grid, FA_THREADS, Fwd3Smem<2>::TOTAL, st>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
