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
//   warp 0    TMA producer: Q once, then K_j / V_j tiles through a 3-slot ring (128B swizzle).
//   warp 1    MMA issuer: S = Q K_j^T (128x128 fp32 in TMEM), then O_j = P_j V_j (128xD in TMEM).
//   warps 2-5 softmax, one query row per thread: read S from TMEM, online max / exp2 / sum, write
//             P_j as bf16 into swizzled shared memory (the A operand of the PV MMA), then fold the
//             block result O_j into the running output kept in registers.
// For D = 64 two CTAs share an SM (96 KB shared memory and 256 TMEM columns each), so one CTA's
// softmax overlaps the other's MMAs. Every wait is bounded and reports through *status.
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
  int* status;
};

template <int ND>
struct FwdSmem {
  static constexpr int TILE = ND * 16384;  // one 128 x (64*ND) bf16 tile
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = TILE;
  static constexpr int P_OFF = KV_OFF + 3 * TILE;
  static constexpr int BAR_OFF = P_OFF + 32768;
  static constexpr int TOTAL = BAR_OFF + 128 + 1024;
};

template <int ND>
__global__ void __launch_bounds__(FA_THREADS, ND == 1 ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const FlashFwdParams p) {
  constexpr int D = 64 * ND;
  using L = FwdSmem<ND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sKV = smem + L::KV_OFF;
  uint8_t* sP = smem + L::P_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;          // 1
  uint64_t* kv_full = bars + 1;     // 3
  uint64_t* kv_empty = bars + 4;    // 3
  uint64_t* s_full = bars + 7;      // 1
  uint64_t* s_empty = bars + 8;     // 1 (128 arrivals)
  uint64_t* p_full = bars + 9;      // 1 (128 arrivals)
  uint64_t* o_full = bars + 10;     // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + FA_BM - 1) / FA_BM;
  const int q_blk = nqb - 1 - blockIdx.x;  // heaviest (latest) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = q_blk * FA_BM;
  const int nkb_all = (p.S + FA_BN - 1) / FA_BN;
  const int nkb = p.causal ? min(nkb_all, q_blk + 1) : nkb_all;
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t O_COL = 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 128);
    mbar_init(p_full, 128);
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
        const int slot = n % 3;
        const uint32_t ph = (n / 3) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&kv_full[slot], L::TILE);
        const int j = n >> 1;
        const CUtensorMap* tm = (n & 1) ? &tmap_v : &tmap_k;
#pragma unroll
        for (int a = 0; a < ND; ++a) tma_load_3d(sKV + slot * L::TILE + a * 16384, tm, &kv_full[slot], hk * D + a * 64, j * FA_BN, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);
      const uint32_t q_base = smem_u32(sQ), p_base = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ERR_WAIT_FULL);
      auto issue_qk = [&](int j) -> bool {
        const int n = 2 * j, slot = n % 3;
        if (!mbar_wait(&kv_full[slot], (n / 3) & 1, abort_flag, p.status, ERR_WAIT_FULL)) return false;
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
        const int n = 2 * j + 1, slot = n % 3;
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status, ERR_WAIT_MISC)) break;
        if (!mbar_wait(&kv_full[slot], (n / 3) & 1, abort_flag, p.status, ERR_WAIT_FULL)) break;
        tc_fence_after();
        const uint32_t v_base = smem_u32(sKV + slot * L::TILE);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          const uint64_t da = make_smem_desc(p_base + (ks / 4) * 16384 + (ks % 4) * 32, 16, 1024, 2);
          const uint64_t db = make_smem_desc(v_base + ks * 2048, 16384, 1024, 2);
          umma_bf16(tmem_base + O_COL, da, db, idesc_pv, ks > 0);
        }
        umma_commit(o_full);
        umma_commit(&kv_empty[slot]);
      }
    }
  } else {
    // ---------------- softmax warps: thread <-> query row ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;  // row inside the tile
    const int row = q0 + r;       // position in the sequence
    const uint32_t t_lane = tmem_base + (uint32_t(q * 32) << 16);
    const float c = p.scale * 1.4426950408889634f;  // fold log2(e) into the scale
    float m = -INFINITY, l = 0.f;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    uint8_t* p_row = sP + (r >> 3) * 1024 + (r & 7) * 128;
    bool ok = true;
    for (int j = 0; j < nkb; ++j) {
      if (!mbar_wait_warp(s_full, j & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * FA_BN;
      const bool need_mask = (p.causal && k0 + FA_BN - 1 > q0) || (k0 + FA_BN > p.S);
      const int kmax = p.causal ? min(row, p.S - 1) : p.S - 1;  // last visible key for this row
      // pass 1: row maximum
      float mx = m;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t rr[32];
        tmem_ld_32x32(t_lane + cc * 32, rr);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (k0 + cc * 32 + i <= kmax) mx = fmaxf(mx, __uint_as_float(rr[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(rr[i]));
        }
      }
      const float m_new = mx;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f((m - m_new) * c);
      const float mc = (m_new == -INFINITY) ? 0.f : m_new * c;
      float rs = 0.f;
      // pass 2: P = exp2(S*c - m*c), written as bf16 into the swizzled A-operand tile
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t rr[32];
        tmem_ld_32x32(t_lane + cc * 32, rr);
        tmem_ld_wait();
        float pv[32];
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float e = exp2f(__uint_as_float(rr[i]) * c - mc);
            if (k0 + cc * 32 + i > kmax) e = 0.f;
            pv[i] = e;
            rs += e;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            pv[i] = exp2f(__uint_as_float(rr[i]) * c - mc);
            rs += pv[i];
          }
        }
        uint8_t* dst = p_row + (cc >> 1) * 16384;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_bf16x2(pv[g * 8 + 0], pv[g * 8 + 1]);
          o.y = pack_bf16x2(pv[g * 8 + 2], pv[g * 8 + 3]);
          o.z = pack_bf16x2(pv[g * 8 + 4], pv[g * 8 + 5]);
          o.w = pack_bf16x2(pv[g * 8 + 6], pv[g * 8 + 7]);
          const int chunk = ((cc & 1) * 4 + g) ^ (r & 7);
          *reinterpret_cast<uint4*>(dst + chunk * 16) = o;
        }
      }
      // S has been read: the next QK^T may overwrite it
      tc_fence_before();
      mbar_arrive(s_empty);
      // P is visible to the tensor core (async proxy) before the PV MMA is released
      fence_proxy_async_smem();
      mbar_arrive(p_full);
      l = l * alpha + rs;
      m = m_new;
      if (!mbar_wait_warp(o_full, j & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t rr[32];
        tmem_ld_32x32(t_lane + O_COL + cc * 32, rr);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[cc * 32 + i] = o_acc[cc * 32 + i] * alpha + __uint_as_float(rr[i]);
      }
      tc_fence_before();
    }
    if (ok && row < p.S) {
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)b * p.S + row) * p.ld_o + h * D;
#pragma unroll
      for (int g = 0; g < D / 8; ++g) {
        uint4 o;
        o.x = pack_bf16x2(o_acc[g * 8 + 0] * inv_l, o_acc[g * 8 + 1] * inv_l);
        o.y = pack_bf16x2(o_acc[g * 8 + 2] * inv_l, o_acc[g * 8 + 3] * inv_l);
        o.z = pack_bf16x2(o_acc[g * 8 + 4] * inv_l, o_acc[g * 8 + 5] * inv_l);
        o.w = pack_bf16x2(o_acc[g * 8 + 6] * inv_l, o_acc[g * 8 + 7] * inv_l);
        *reinterpret_cast<uint4*>(dst + g * 8) = o;
      }
      if (p.lse) p.lse[((size_t)b * p.H + h) * p.S + row] = m * c + log2f(l);  // log2 domain, consumed by the backward
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

// ------------------------------------------------------------------------------------------------
// Second-generation forward kernel (the default). Same roles and ring as above; what changed is the
// softmax / accumulation scheme, which is where the first kernel spent its time:
//   * O stays in TMEM for the whole key loop: every PV MMA accumulates into it. The running maximum
//     is only raised when a block's maximum exceeds it by more than 8 (log2 units), so the rescale of
//     O (TMEM load, multiply, TMEM store) is rare after the first blocks; until then P may reach 2^8,
//     which bf16 / fp32 hold without loss.
//   * the row sums are produced by the tensor core too: a second, 16-column MMA multiplies P by a tile
//     of ones, so l accumulates next to O in TMEM from exactly the bf16 values the PV MMA consumed.
//   * exponentials run two per MUFU instruction on packed bf16 (cvt.rn.bf16x2 + ex2.approx.bf16x2),
//     whose result is already the A-operand format; the row maximum uses 3-input max with four
//     independent chains.
// ------------------------------------------------------------------------------------------------
template <int ND>
struct Fwd2Smem {
  static constexpr int TILE = ND * 16384;
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = TILE;
  static constexpr int P_OFF = KV_OFF + 3 * TILE;
  static constexpr int ONES_OFF = P_OFF + 32768;      // 16 rows x 128 keys of bf16 1.0 (K-major, any swizzle: all equal)
  static constexpr int BAR_OFF = ONES_OFF + 4096;
  static constexpr int TOTAL = BAR_OFF + 128 + 1024;
};

template <int ND>
__global__ void __launch_bounds__(FA_THREADS, ND == 1 ? 2 : 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const FlashFwdParams p) {
  constexpr int D = 64 * ND;
  using L = Fwd2Smem<ND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sKV = smem + L::KV_OFF;
  uint8_t* sP = smem + L::P_OFF;
  uint8_t* sOnes = smem + L::ONES_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;          // 1
  uint64_t* kv_full = bars + 1;     // 3
  uint64_t* kv_empty = bars + 4;    // 3
  uint64_t* s_full = bars + 7;      // 1
  uint64_t* s_empty = bars + 8;     // 1 (128 arrivals)
  uint64_t* p_full = bars + 9;      // 1 (128 arrivals)
  uint64_t* o_full = bars + 10;     // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + FA_BM - 1) / FA_BM;
  const int q_blk = nqb - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = q_blk * FA_BM;
  const int nkb_all = (p.S + FA_BN - 1) / FA_BN;
  const int nkb = p.causal ? min(nkb_all, q_blk + 1) : nkb_all;
  constexpr uint32_t TMEM_COLS = ND == 1 ? 256 : 512;
  constexpr uint32_t O_COL = 128, L_COL = 128 + D;

  for (int i = threadIdx.x; i < 4096 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(sOnes)[i] = 0x3f803f80u;  // bf16 1.0 pairs
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 128);
    mbar_init(p_full, 128);
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
  fence_proxy_async_smem();  // the ones tile is read by the tensor core
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
        const int slot = n % 3;
        const uint32_t ph = (n / 3) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&kv_full[slot], L::TILE);
        const int j = n >> 1;
        const CUtensorMap* tm = (n & 1) ? &tmap_v : &tmap_k;
#pragma unroll
        for (int a = 0; a < ND; ++a) tma_load_3d(sKV + slot * L::TILE + a * 16384, tm, &kv_full[slot], hk * D + a * 64, j * FA_BN, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);
      const uint32_t idesc_l = make_idesc_bf16(128, 16, 0, 0);
      const uint32_t q_base = smem_u32(sQ), p_base = smem_u32(sP), ones_base = smem_u32(sOnes);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ERR_WAIT_FULL);
      auto issue_qk = [&](int j) -> bool {
        const int n = 2 * j, slot = n % 3;
        if (!mbar_wait(&kv_full[slot], (n / 3) & 1, abort_flag, p.status, ERR_WAIT_FULL)) return false;
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
        const int n = 2 * j + 1, slot = n % 3;
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status, ERR_WAIT_MISC)) break;
        if (!mbar_wait(&kv_full[slot], (n / 3) & 1, abort_flag, p.status, ERR_WAIT_FULL)) break;
        tc_fence_after();
        const uint32_t v_base = smem_u32(sKV + slot * L::TILE);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          const uint64_t da = make_smem_desc(p_base + (ks / 4) * 16384 + (ks % 4) * 32, 16, 1024, 2);
          const uint64_t db = make_smem_desc(v_base + ks * 2048, 16384, 1024, 2);
          const uint32_t acc = (j > 0 || ks > 0) ? 1u : 0u;
          umma_bf16(tmem_base + O_COL, da, db, idesc_pv, acc);
          umma_bf16(tmem_base + L_COL, da, make_smem_desc(ones_base + (ks / 4) * 2048 + (ks % 4) * 32, 16, 1024, 2), idesc_l, acc);
        }
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
    float m_used = -INFINITY;  // the maximum the exponentials are taken against (scores, not yet scaled by c)
    uint8_t* p_row = sP + (r >> 3) * 1024 + (r & 7) * 128;
    bool ok = true;
    for (int j = 0; j < nkb; ++j) {
      if (!mbar_wait_warp(s_full, j & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * FA_BN;
      const bool need_mask = (p.causal && k0 + FA_BN - 1 > q0) || (k0 + FA_BN > p.S);
      const int kmax = p.causal ? min(row, p.S - 1) : p.S - 1;
      // the whole score row moves into registers with four back-to-back TMEM loads and one wait (the load latency
      // is paid once per block, not once per 32 columns), and S is handed back to the tensor core right away
      uint32_t sr[128];
      tmem_ld_32x32(t_lane, sr);
      tmem_ld_32x32(t_lane + 32, sr + 32);
      tmem_ld_32x32(t_lane + 64, sr + 64);
      tmem_ld_32x32(t_lane + 96, sr + 96);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_empty);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (k0 + i > kmax) sr[i] = 0xff800000u;  // -inf
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
      // raise the working maximum only when the block exceeds it by more than 2^8
      const bool raise = j == 0 || (m_blk - m_used) * c > 8.0f;
      const float m_new = raise ? fmaxf(m_used, m_blk) : m_used;
      const float alpha = (j == 0 || !raise) ? 1.0f : exp2f((m_used - m_new) * c);
      m_used = m_new;
      const bool any_rescale = __any_sync(0xffffffffu, j > 0 && raise);
      if (j > 0) {
        // PV of the previous block is complete: the P buffer is free and O / l are stable
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
          uint32_t ll[16];
          tmem_ld_32x16(t_lane + L_COL, ll);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) ll[i] = __float_as_uint(__uint_as_float(ll[i]) * alpha);
          tmem_st_32x16(t_lane + L_COL, ll);
          tmem_st_wait();
          tc_fence_before();
        }
      }
      const float mc = m_used * c;
      // P = exp2(S*c - m*c) as packed bf16 straight into the swizzled A-operand tile
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          pk[i] = ex2_bf16x2(cvt_bf16x2(fmaf(__uint_as_float(sr[cc * 32 + 2 * i]), c, -mc), fmaf(__uint_as_float(sr[cc * 32 + 2 * i + 1]), c, -mc)));
        uint8_t* dst = p_row + (cc >> 1) * 16384;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = ((cc & 1) * 4 + g) ^ (r & 7);
          *reinterpret_cast<uint4*>(dst + chunk * 16) = make_uint4(pk[g * 4 + 0], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(p_full);
    }
    if (ok) ok = mbar_wait_warp(o_full, (nkb - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      uint32_t ll[16];
      tmem_ld_32x16(t_lane + L_COL, ll);
      tmem_ld_wait();
      const float l = __uint_as_float(ll[0]);
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

// ------------------------------------------------------------------------------------------------
// Third-generation forward kernel (the default). Cycle stamps of the second generation showed where a
// key block's ~4000 cycles went: ~1500 waiting for a K tile (three ring slots: the load of K_{j+1} could
// not start before P_{j-1}V_{j-1} had finished), ~1000 waiting for the previous PV MMA before the
// exponentials even started, ~1200 in the PV MMA plus a separate row-sum MMA, and ~1800 in the
// exponential phase itself (MUFU-bound). This version
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
  const int nkb = p.causal ? min(nkb_all, q_blk + 1) : nkb_all;
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
        const int j = n >> 1;
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
      const int k0 = j * FA_BN;
      const bool need_mask = (p.causal && k0 + FA_BN - 1 > q0) || (k0 + FA_BN > p.S);
      const int kmax = p.causal ? min(row, p.S - 1) : p.S - 1;
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
          if (k0 + i > kmax) sr[i] = 0xff800000u;  // -inf
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
      const float mc = m_used * c;
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

}  // namespace inv

using namespace inv;

// q/k/v: token-major bf16 [B*S, ld*]; q has H heads, k and v have Hkv heads of `head_dim` columns.
// out: [B*S, ld_o] bf16; lse: [B, H, S] fp32 (may be null).
extern "C" int inv_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int H, int Hkv,
                                  int head_dim, int ld_q, int ld_k, int ld_v, int ld_o, float scale, int causal, int* status, void* stream) {
  if ((head_dim != 64 && head_dim != 128) || H % Hkv || (ld_q % 8) || (ld_k % 8) || (ld_v % 8) || (ld_o % 8)) return -ERR_BAD_ARG;
  if (B <= 0 || S <= 0) return 0;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_tokens_bf16(&tq, q, H * head_dim, S, B, ld_q, FA_BM))) return rc;
  if ((rc = make_tmap_tokens_bf16(&tk, k, Hkv * head_dim, S, B, ld_k, FA_BN))) return rc;
  if ((rc = make_tmap_tokens_bf16(&tv, v, Hkv * head_dim, S, B, ld_v, FA_BN))) return rc;
  FlashFwdParams p;
  p.out = (__nv_bfloat16*)out; p.ld_o = ld_o; p.lse = lse;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv; p.scale = scale; p.causal = causal; p.status = status;
  dim3 grid((S + FA_BM - 1) / FA_BM, H, B);
  cudaStream_t st = (cudaStream_t)stream;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(flash_fwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<1>::TOTAL);
    cudaFuncSetAttribute(flash_fwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<2>::TOTAL);
    cudaFuncSetAttribute(flash_fwd2_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Smem<1>::TOTAL);
    cudaFuncSetAttribute(flash_fwd2_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Smem<2>::TOTAL);
    cudaFuncSetAttribute(flash_fwd3_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd3Smem<1>::TOTAL);
    cudaFuncSetAttribute(flash_fwd3_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd3Smem<2>::TOTAL);
    configured = true;
  }
  const bool legacy = (causal & 8) != 0;  // bit 3 selects the first-generation kernel, bit 5 the second (A/B comparisons)
  const bool gen2 = (causal & 32) != 0;
  p.causal = causal & 1;
  if (gen2) {
    if (head_dim == 64) flash_fwd2_kernel<1><<<grid, FA_THREADS, Fwd2Smem<1>::TOTAL, st>>>(tq, tk, tv, p);
    else flash_fwd2_kernel<2><<<grid, FA_THREADS, Fwd2Smem<2>::TOTAL, st>>>(tq, tk, tv, p);
  } else if (legacy) {
    if (head_dim == 64) flash_fwd_kernel<1><<<grid, FA_THREADS, FwdSmem<1>::TOTAL, st>>>(tq, tk, tv, p);
    else flash_fwd_kernel<2><<<grid, FA_THREADS, FwdSmem<2>::TOTAL, st>>>(tq, tk, tv, p);
  } else {
    if (head_dim == 64) flash_fwd3_kernel<1><<<grid, FA_THREADS, Fwd3Smem<1>::TOTAL, st>>>(tq, tk, tv, p);
    else flash_fwd3_kernel<2><<<grid, FA_THREADS, Fwd3Smem<2>::TOTAL, st>>>(tq, tk, tv, p);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
