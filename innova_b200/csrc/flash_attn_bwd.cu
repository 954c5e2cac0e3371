// Flash attention backward on tcgen05 tensor cores (causal or full, MHA or GQA, head_dim 64 or 128).
//
// Replaces the reference's attention backward (include/oil/autograd_functions.h:82-94,
// src/autograd_grad.cpp attention branch); the reference's memory-efficient backward is a
// placeholder (src/zero_optimizer_mem.cpp:496-574), so the oracle is plain fp32 attention.
//
// One CTA per (batch, kv head, 128-key block). K and V tiles stay in shared memory; the CTA walks
// the query blocks that can see its keys (and, for GQA, every query head of the group) and
// accumulates dK and dV in TMEM. Per query block, five MMAs:
//   S^T  = K Q^T            dP^T = V dO^T            (both 128 keys x 128 queries, fp32 in TMEM)
//   dV  += P^T dO           dK  += dS^T Q            dQ_blk = dS K
// 16 softmax warps (thread <-> key row, four quarters of the query columns) turn S^T, dP^T into
// P^T = exp(S^T*scale - lse) and dS^T = P^T * (dP^T - D) as bf16 tiles in swizzled shared memory.
// The same dS^T tile serves as a K-major A operand (dK) and as an MN-major A operand (dQ), and the
// Q / dO / K tiles serve as K-major B operands (S^T, dP^T) and MN-major B operands (dK, dV, dQ), so
// nothing is transposed in memory. dQ blocks are added to an fp32 buffer with vector reductions.
// Every wait is bounded and reports through *status.
#include "sm100_common.cuh"
#include "inv_api.h"

#include <type_traits>

namespace inv {

int make_tmap_tokens_bf16(CUtensorMap* out, const void* ptr, int cols, int S, int B, int ld, int box_rows);
int make_tmap_tokens_f32(CUtensorMap* out, const void* ptr, int cols, int S, int B);

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }  // sources read
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }        // copies complete
// Adds a shared-memory box (shape and swizzle are the tensor map's: 32 rows x 16 floats, 64-byte swizzle) into the fp32
// tensor behind the map. Rows past the end of a sequence are clipped by the copy engine.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}

constexpr int FB_THREADS = 640;  // warp 0 TMA, warps 1, 18, 19 MMA issuers, warps 2-17 softmax (four per scheduler: the
                                 // dependent FMA -> MUFU -> FMUL -> convert chains of two warps per scheduler left it mostly idle)

struct FlashBwdParams {
  const float* lse;    // [B, H, S], log2 domain: log2(sum exp(scores))
  const float* delta;  // [B, H, S]  rowsum(dO * O)
  float* dq_acc;       // [B*S, H*D] fp32, zero on entry
  __nv_bfloat16* dk;   // token-major, ld_dk
  __nv_bfloat16* dv;
  int ld_dk, ld_dv;
  int B, S, H, Hkv;
  float scale;
  int causal;
  int window;  // > 0 (causal only): a query sees the `window` most recent keys, its own position included
  int* status;
};

template <int ND>
struct BwdSmem {
  static constexpr int TILE = ND * 16384;
  static constexpr int STAGES = ND == 1 ? 2 : 1;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int Q_OFF = 2 * TILE;
  static constexpr int DO_OFF = Q_OFF + STAGES * TILE;
  static constexpr int PT_OFF = DO_OFF + STAGES * TILE;
  static constexpr int DST_OFF = PT_OFF + 32768;
  static constexpr int DQS_OFF = DST_OFF + 32768;      // D = 64: the fp32 dQ block on its way to the reduce copies, one 32 x 16 box per softmax warp
  static constexpr int STAT_OFF = DQS_OFF + (ND == 1 ? 32768 : 0);  // lse and delta of the current query block, two stages
  static constexpr int BAR_OFF = STAT_OFF + 16 * 2 * 64 * 4;   // per softmax warp: two stages of 32 lse + 32 delta
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// Build with -DFB_TRACE to record the SM clock at the phases of CTA (0, 0, 0) of the most recent launch
// (inv_fb_trace_read): 0 entry, 1 set-up done, 2 K/V landed (issuer), 3 exit, 4 dK/dV written, 8 + 3 it: S^T ready for
// query block it, 9 + 3 it: P^T / dS^T published, 10 + 3 it: dQ of block it - 1 read out, 32 + 3 it: S^T / dP^T in registers,
// 33 + 3 it: exponentials done, 34 + 3 it: the previous block's MMAs have released the P^T / dS^T tiles.
#ifdef FB_TRACE
__device__ long long fb_trace_buf[64];
#define FB_STAMP(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (i) < 64) fb_trace_buf[i] = clock64(); } while (0)
#else
#define FB_STAMP(i) do {} while (0)
#endif

template <int ND>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                 const __grid_constant__ CUtensorMap tmap_dq, const FlashBwdParams p) {
  constexpr int D = 64 * ND;
  constexpr bool DQ_TMA = (ND == 1);  // dQ blocks leave through shared memory and one reduce copy per 32 columns, not per-thread reductions
  using L = BwdSmem<ND>;
  constexpr int STAGES = L::STAGES;
  constexpr bool OVERLAP = (ND == 1);  // D = 128 has no spare TMEM: dQ reuses the S^T columns
  constexpr uint32_t ST_COL = 0, DPT_COL = 128, DV_COL = 256, DK_COL = 256 + D, DQ_COL = OVERLAP ? 384 : 0;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::K_OFF;
  uint8_t* sV = smem + L::V_OFF;
  uint8_t* sQ = smem + L::Q_OFF;
  uint8_t* sdO = smem + L::DO_OFF;
  uint8_t* sPt = smem + L::PT_OFF;
  uint8_t* sdSt = smem + L::DST_OFF;
  uint8_t* sDq = smem + L::DQS_OFF;
  float* sStat = reinterpret_cast<float*>(smem + L::STAT_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;        // 1
  uint64_t* q_full = bars + 1;     // STAGES
  uint64_t* q_empty = bars + 3;    // STAGES
  uint64_t* s_full = bars + 5;     // S^T and dP^T are in TMEM
  uint64_t* s_empty = bars + 6;    // 256 arrivals: both have been read
  uint64_t* pds_full = bars + 7;   // 256 arrivals: P^T and dS^T are in shared memory
  uint64_t* mma2_done = bars + 8;  // dV, dK, dQ MMAs of this block finished
  uint64_t* dq_empty = bars + 9;   // 256 arrivals: dQ has been read out of TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int k0 = j * 128;
  const int nqb = (p.S + 127) / 128;
  const int i0 = p.causal ? j : 0;
  // with a sliding window the last query that sees key k0 + 127 is row k0 + 126 + window
  const int i_end = (p.causal && p.window > 0) ? min(nqb, (k0 + 126 + p.window) / 128 + 1) : nqb;
  const int nq_it = i_end - i0;
  const int n_it = G * nq_it;
  if (threadIdx.x == 0) FB_STAMP(0);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 2);  // the two issuers that read Q and dO
    }
    mbar_init(s_full, 2);      // S^T and dP^T have one issuer each
    mbar_init(s_empty, 16);
    mbar_init(pds_full, 16);
    mbar_init(mma2_done, 3);   // dV, dK and dQ have one issuer each
    mbar_init(dq_empty, 16);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
    if (DQ_TMA) tma_prefetch_desc(&tmap_dq);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) FB_STAMP(1);

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
      for (int a = 0; a < ND; ++a) {
        tma_load_3d(sK + a * 16384, &tmap_k, kv_full, hk * D + a * 64, k0, b);
        tma_load_3d(sV + a * 16384, &tmap_v, kv_full, hk * D + a * 64, k0, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&q_empty[st], ph ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) break;
        const int h = hk * G + it / nq_it;
        const int q0 = (i0 + it % nq_it) * 128;
        mbar_expect_tx(&q_full[st], 2 * L::TILE);
#pragma unroll
        for (int a = 0; a < ND; ++a) {
          tma_load_3d(sQ + st * L::TILE + a * 16384, &tmap_q, &q_full[st], h * D + a * 64, q0, b);
          tma_load_3d(sdO + st * L::TILE + a * 16384, &tmap_do, &q_full[st], h * D + a * 64, q0, b);
        }
      }
    }
  } else if (warp == 1 || warp >= 18) {
    // Three MMA issuers in three warps. A thread issues one tcgen05.mma per ~100 cycles whatever its size, and a
    // query block needs 32 (D = 64) or 64 of them: one issuer would spend more time issuing than the tensor pipe
    // spends computing. Every accumulator has exactly one issuer, so the order of its updates is program order:
    //   role 0 (warp 1):  S^T = K Q^T    and  dV += P^T dO
    //   role 1 (warp 18): dP^T = V dO^T  and  dK += dS^T Q
    //   role 2 (warp 19): dQ_blk = dS K
    if (lane == 0) {
      const int role = warp == 1 ? 0 : warp - 17;
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // K-major x K-major
      const uint32_t idesc_kv = make_idesc_bf16(128, D, 0, 1);    // K-major A, MN-major B
      const uint32_t idesc_dq = make_idesc_bf16(128, D, 1, 1);    // MN-major A and B
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV);
      const uint32_t pt_base = smem_u32(sPt), dst_base = smem_u32(sdSt);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, ERR_WAIT_FULL);
      if (role == 0) FB_STAMP(2);
      auto issue_s = [&](int it) -> bool {  // roles 0 and 1
        const int st = it % STAGES;
        if (!mbar_wait(&q_full[st], (it / STAGES) & 1, abort_flag, p.status, ERR_WAIT_FULL)) return false;
        if (it > 0 && !mbar_wait(s_empty, (it - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) return false;
        if (!OVERLAP && role == 0 && it > 0 && !mbar_wait(dq_empty, (it - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t a_base = role == 0 ? k_base : v_base;
        const uint32_t b_base = smem_u32((role == 0 ? sQ : sdO) + st * L::TILE);
        const uint32_t d_col = tmem_base + (role == 0 ? ST_COL : DPT_COL);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
          umma_bf16(d_col, make_smem_desc(a_base + off, 16, 1024, 2), make_smem_desc(b_base + off, 16, 1024, 2), idesc_s, ks > 0);
        }
        umma_commit(s_full);
        return true;
      };
      if (ok && OVERLAP && role < 2) ok = issue_s(0);
      for (int it = 0; ok && it < n_it; ++it) {
        if (role < 2) {
          if (OVERLAP) {
            if (it + 1 < n_it && !issue_s(it + 1)) break;
          } else {
            if (!issue_s(it)) break;
          }
        }
        const int st = it % STAGES;
        if (!mbar_wait(pds_full, it & 1, abort_flag, p.status, ERR_WAIT_MISC)) break;
        if (OVERLAP && role == 2 && it > 0 && !mbar_wait(dq_empty, (it - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        if (role < 2) {
          // dV += P^T dO ; dK += dS^T Q   (A: [keys x queries] K-major, B: [queries x d] MN-major)
          const uint32_t a_base = role == 0 ? pt_base : dst_base;
          const uint32_t b_base = smem_u32((role == 0 ? sdO : sQ) + st * L::TILE);
          const uint32_t d_col = tmem_base + (role == 0 ? DV_COL : DK_COL);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a_off = (ks / 4) * 16384 + (ks % 4) * 32;
            umma_bf16(d_col, make_smem_desc(a_base + a_off, 16, 1024, 2), make_smem_desc(b_base + ks * 2048, 16384, 1024, 2), idesc_kv,
                      (it > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(mma2_done);
          umma_commit(&q_empty[st]);  // both roles read Q and dO of this stage
        } else {
          // dQ_blk = dS K   (A: dS^T tile read MN-major, B: K tile read MN-major; reduction over keys)
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            umma_bf16(tmem_base + DQ_COL, make_smem_desc(dst_base + ks * 2048, 16384, 1024, 2), make_smem_desc(k_base + ks * 2048, 16384, 1024, 2),
                      idesc_dq, ks > 0);
          }
          umma_commit(mma2_done);
        }
      }
    }
  } else if (warp >= 2 && warp < 18) {
    // ---------------- softmax warps ----------------
    const int q = warp & 3;            // TMEM lane quarter
    const int cq = (warp - 2) >> 2;    // which quarter of the 128 query columns (32 per thread)
    const int hf = cq >> 1;            // the 64-column half (shared-memory tile) it falls in
    constexpr int DC = D / 4;          // dQ / dK / dV columns per thread
    const int r = q * 32 + lane;       // row inside a tile
    const int key = k0 + r;
    const uint32_t t_lane = tmem_base + (uint32_t(q * 32) << 16);
    const float c = p.scale * 1.4426950408889634f;
    const bool vec_ok = (p.S & 3) == 0;  // rows of lse / delta start 16-byte aligned
    uint8_t* pt_row = sPt + hf * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
    uint8_t* dst_row = sdSt + hf * 16384 + (r >> 3) * 1024 + (r & 7) * 128;
    bool ok = true;
    // dQ block j: TMEM lanes are query rows now; this thread adds D/2 columns of row q0 + r into the fp32 buffer
    auto dq_readout = [&](int j) {
      const int hj = hk * G + j / nq_it;
      const int qrow = (i0 + j % nq_it) * 128 + r;
      if (DQ_TMA) {
        // Every warp drains its own 32 rows x 16 columns: TMEM -> a private 2 KB box in shared memory (64-byte rows,
        // 64-byte swizzle: chunk ^ ((row >> 1) & 3)) -> one reduce copy issued by the warp's first lane. No barrier
        // across warps: a warp only waits for its own previous copy to have read its box.
        uint32_t rr[16];
        tmem_ld_32x16(t_lane + DQ_COL + cq * 16, rr);
        if (lane == 0) bulk_wait_read();
        __syncwarp();
        tmem_ld_wait();
        uint8_t* box = sDq + (warp - 2) * 2048;
        uint8_t* row = box + lane * 64;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = g ^ ((lane >> 1) & 3);
          *reinterpret_cast<uint4*>(row + chunk * 16) = make_uint4(rr[g * 4], rr[g * 4 + 1], rr[g * 4 + 2], rr[g * 4 + 3]);
        }
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(dq_empty);
          tma_reduce_add_3d(&tmap_dq, box, hj * D + cq * 16, (i0 + j % nq_it) * 128 + q * 32, b);
          bulk_commit();
        }
        return;
      }
      {
        const int col0 = cq * DC;
        uint32_t rr[DC];
        if (DC == 16) tmem_ld_32x16(t_lane + DQ_COL + col0, rr);
        else tmem_ld_32x32(t_lane + DQ_COL + col0, rr);
        tmem_ld_wait();
        if (qrow < p.S) {
          float* dst = p.dq_acc + ((size_t)b * p.S + qrow) * ((size_t)p.H * D) + hj * D + col0;
#pragma unroll
          for (int g = 0; g < DC / 4; ++g)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + g * 4), "f"(__uint_as_float(rr[g * 4])),
                         "f"(__uint_as_float(rr[g * 4 + 1])), "f"(__uint_as_float(rr[g * 4 + 2])), "f"(__uint_as_float(rr[g * 4 + 3]))
                         : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);
    };
    // The row statistics (lse, delta) of a query block go through shared memory, a private region per warp: lane i
    // fetches lse and delta of column cq * 32 + i (two global loads per thread and block; the four warps of a column
    // quarter fetch the same values), the inner loop reads them back as broadcast 16-byte loads. The loads for block
    // it + 1 are issued while block it is being computed and parked in registers, so that no warp waits on them, and
    // no barrier across warps is involved.
    float* wstat = sStat + (warp - 2) * 128;  // [stage][lse 32 | delta 32]
    auto stat_load = [&](int it, float& l, float& d) {
      const int h = hk * G + it / nq_it;
      const int qi = min((i0 + it % nq_it) * 128 + cq * 32 + lane, p.S - 1);
      const size_t o = ((size_t)b * p.H + h) * p.S + qi;
      l = __ldg(p.lse + o);
      d = __ldg(p.delta + o);
    };
    if (n_it > 0) {
      float l, d;
      stat_load(0, l, d);
      wstat[lane] = l;
      wstat[32 + lane] = d;
    }
    for (int it = 0; it < n_it; ++it) {
      const int q0 = (i0 + it % nq_it) * 128;
      const float* stat = wstat + (it & 1) * 64;
      if (!mbar_wait_warp(s_full, it & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      if (threadIdx.x == 64) FB_STAMP(8 + 3 * it);
      __syncwarp();  // the statistics of this block are in place (written by this warp)
      const bool windowed = p.causal && p.window > 0;
      const bool need_mask = (p.causal && q0 < k0 + 127) || (q0 + 128 > p.S) || (k0 + 128 > p.S) || (windowed && q0 + 127 - k0 >= p.window);
      // The thread's 32 columns of S^T and dP^T come in as two halves of 16 (the register file holds 96 registers per
      // thread at this block size: both halves at once spill). The TMEM columns go back to the tensor core after the
      // second load. A column i of the thread is live iff lim_lo <= i < lim_hi (causal diagonal, sequence end, window).
      uint32_t pk[16], dk[16];  // P^T and dS^T of this thread's 32 columns as packed bf16 pairs, kept in registers until the
                                // shared-memory tiles are free
      float stat_next_l = 0.f, stat_next_d = 0.f;
      const int col0 = cq * 32;
      int lim_lo = 0, lim_hi = 32;
      if (need_mask) {
        if (p.causal) lim_lo = key - q0 - col0;
        lim_hi = min(32, p.S - q0 - col0);
        if (windowed) lim_hi = min(lim_hi, key + p.window - q0 - col0);
        if (key >= p.S) lim_hi = 0;
      }
      auto softmax_block = [&](auto masked_tag) {
      constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t s_r[16], dp_r[16];
        tmem_ld_32x16(t_lane + ST_COL + col0 + half * 16, s_r);
        tmem_ld_32x16(t_lane + DPT_COL + col0 + half * 16, dp_r);
        tmem_ld_wait();
        if (half == 1) {
          if (threadIdx.x == 64) FB_STAMP(32 + 3 * it);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty);  // one arrival per warp: arrivals on one mbarrier are serialised
          if (it + 1 < n_it) stat_load(it + 1, stat_next_l, stat_next_d);
        }
        // statistics as 16-byte broadcast loads; one MUFU op and half a conversion per element
        const float4* l4 = reinterpret_cast<const float4*>(stat + half * 16);
        const float4* d4 = reinterpret_cast<const float4*>(stat + 32 + half * 16);
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
          const float4 l = l4[i4], dl = d4[i4];
          const int i = i4 * 4;
          float e0 = exp2f(fmaf(__uint_as_float(s_r[i]), c, -l.x)), e1 = exp2f(fmaf(__uint_as_float(s_r[i + 1]), c, -l.y));
          float e2 = exp2f(fmaf(__uint_as_float(s_r[i + 2]), c, -l.z)), e3 = exp2f(fmaf(__uint_as_float(s_r[i + 3]), c, -l.w));
          if (MASKED) {
            const int ci = half * 16 + i;
            e0 = (ci >= lim_lo && ci < lim_hi) ? e0 : 0.f;
            e1 = (ci + 1 >= lim_lo && ci + 1 < lim_hi) ? e1 : 0.f;
            e2 = (ci + 2 >= lim_lo && ci + 2 < lim_hi) ? e2 : 0.f;
            e3 = (ci + 3 >= lim_lo && ci + 3 < lim_hi) ? e3 : 0.f;
          }
          const int o = half * 8 + i4 * 2;
          pk[o] = cvt_bf16x2(e0, e1);
          pk[o + 1] = cvt_bf16x2(e2, e3);
          dk[o] = cvt_bf16x2(e0 * (__uint_as_float(dp_r[i]) - dl.x), e1 * (__uint_as_float(dp_r[i + 1]) - dl.y));
          dk[o + 1] = cvt_bf16x2(e2 * (__uint_as_float(dp_r[i + 2]) - dl.z), e3 * (__uint_as_float(dp_r[i + 3]) - dl.w));
        }
      }
      };
      if (need_mask) softmax_block(std::true_type{});   // two copies of the loop: interior blocks carry no selects
      else softmax_block(std::false_type{});
      // the warp's other statistics stage was last read in block it - 1
      if (it + 1 < n_it) {
        wstat[((it + 1) & 1) * 64 + lane] = stat_next_l;
        wstat[((it + 1) & 1) * 64 + 32 + lane] = stat_next_d;
      }
      // Software pipeline (when dQ has its own TMEM columns): the arithmetic above ran while the MMAs of the previous
      // block were still reading its P^T / dS^T tiles; only now wait for them, publish this block's tiles, and read the
      // previous block's dQ out of TMEM while this block's MMAs run.
      if (threadIdx.x == 64) FB_STAMP(33 + 3 * it);
      if (OVERLAP && it > 0) {
        if (!mbar_wait_warp(mma2_done, (it - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
      }
      if (threadIdx.x == 64) FB_STAMP(34 + 3 * it);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int chunk = ((cq & 1) * 4 + g) ^ (r & 7);
        *reinterpret_cast<uint4*>(pt_row + chunk * 16) = make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
        *reinterpret_cast<uint4*>(dst_row + chunk * 16) = make_uint4(dk[g * 4], dk[g * 4 + 1], dk[g * 4 + 2], dk[g * 4 + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (threadIdx.x == 64) FB_STAMP(9 + 3 * it);
      if (OVERLAP) {
        if (it > 0) dq_readout(it - 1);
        if (threadIdx.x == 64) FB_STAMP(10 + 3 * it);
      } else {
        if (!mbar_wait_warp(mma2_done, it & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        dq_readout(it);
      }
    }
    if (OVERLAP && ok && n_it > 0) {
      if (mbar_wait_warp(mma2_done, (n_it - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) {
        tc_fence_after();
        dq_readout(n_it - 1);
      } else {
        ok = false;
      }
    }
    // dK, dV: the last mma2_done covers every accumulation. TMEM lanes are key rows.
    if (ok && n_it > 0) {
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t colbase = which == 0 ? DV_COL : DK_COL;
        __nv_bfloat16* outp = which == 0 ? p.dv : p.dk;
        const int ld = which == 0 ? p.ld_dv : p.ld_dk;
        const float sc = which == 0 ? 1.f : p.scale;
        {
          const int col0 = cq * DC;
          uint32_t rr[DC];
          if (DC == 16) tmem_ld_32x16(t_lane + colbase + col0, rr);
          else tmem_ld_32x32(t_lane + colbase + col0, rr);
          tmem_ld_wait();
          if (key < p.S) {
            __nv_bfloat16* dst = outp + ((size_t)b * p.S + key) * ld + hk * D + col0;
#pragma unroll
            for (int g = 0; g < DC / 8; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(rr[g * 8 + 0]) * sc, __uint_as_float(rr[g * 8 + 1]) * sc);
              o.y = pack_bf16x2(__uint_as_float(rr[g * 8 + 2]) * sc, __uint_as_float(rr[g * 8 + 3]) * sc);
              o.z = pack_bf16x2(__uint_as_float(rr[g * 8 + 4]) * sc, __uint_as_float(rr[g * 8 + 5]) * sc);
              o.w = pack_bf16x2(__uint_as_float(rr[g * 8 + 6]) * sc, __uint_as_float(rr[g * 8 + 7]) * sc);
              *reinterpret_cast<uint4*>(dst + g * 8) = o;
            }
          }
        }
      }
      tc_fence_before();
      if (threadIdx.x == 64) FB_STAMP(4);
    }
    if (DQ_TMA && lane == 0) bulk_wait_all();  // this warp's reduce copies must have landed before the grid ends
  }

  __syncthreads();
  if (threadIdx.x == 0) FB_STAMP(3);
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

// delta[b,h,s] = sum_d O[b,s,h,d] * dO[b,s,h,d]. One warp per 32/(D/8) (token, head) pairs.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta, int B,
                                  int S, int H, int D, int ld_o, int ld_do) {
  const int lanes_per = D / 8;  // 8 or 16
  const long gid = blockIdx.x * (long)blockDim.x + threadIdx.x;
  const long pair = gid / lanes_per;
  const int v = (int)(gid % lanes_per);
  const long total = (long)B * S * H;
  float s = 0.f;
  if (pair < total) {
    const int h = (int)(pair % H);
    const long t = pair / H;
    uint4 a = *reinterpret_cast<const uint4*>(o + t * ld_o + h * D + v * 8);
    uint4 g = *reinterpret_cast<const uint4*>(d_o + t * ld_do + h * D + v * 8);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(g2[i]);
      s += x.x * y.x + x.y * y.y;
    }
  }
  for (int off = lanes_per / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (pair < total && v == 0) {
    const int h = (int)(pair % H);
    const long t = pair / H;
    const long bb = t / S, ss = t % S;
    delta[(bb * H + h) * S + ss] = s;
  }
}

// dq[t, :] = bf16(dq_acc[t, :] * scale), written into a token-major buffer with row pitch ld.
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long T, int cols, int ld, float scale) {
  const int vec = cols / 8;
  const long total = T * vec;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / vec;
    const int cidx = (int)(i % vec) * 8;
    const float4 a = *reinterpret_cast<const float4*>(acc + t * cols + cidx);
    const float4 b2 = *reinterpret_cast<const float4*>(acc + t * cols + cidx + 4);
    uint4 o;
    o.x = pack_bf16x2(a.x * scale, a.y * scale);
    o.y = pack_bf16x2(a.z * scale, a.w * scale);
    o.z = pack_bf16x2(b2.x * scale, b2.y * scale);
    o.w = pack_bf16x2(b2.z * scale, b2.w * scale);
    *reinterpret_cast<uint4*>(dq + t * ld + cidx) = o;
  }
}

}  // namespace inv

using namespace inv;

// Scratch needed by inv_flash_attn_bwd: delta [B,H,S] fp32 followed by dq_acc [B*S, H*D] fp32.
extern "C" long inv_flash_attn_bwd_scratch_bytes(int B, int S, int H, int head_dim) {
  long delta = (((long)B * H * S * 4) + 255) & ~255L;
  return delta + (long)B * S * H * head_dim * 4;
}

// q,k,v,o,do: token-major bf16. dq,dk,dv: token-major bf16 outputs (may point into one dqkv buffer).
extern "C" int inv_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, void* dq,
                                  void* dk, void* dv, void* scratch, int B, int S, int H, int Hkv, int head_dim, int ld_q, int ld_k, int ld_v,
                                  int ld_o, int ld_do, int ld_dq, int ld_dk, int ld_dv, float scale, int causal, int window, int* status,
                                  void* stream) {
  if ((head_dim != 64 && head_dim != 128) || H % Hkv || (ld_q % 8) || (ld_k % 8) || (ld_v % 8) || (ld_o % 8) || (ld_do % 8) ||
      (ld_dq % 8) || (ld_dk % 8) || (ld_dv % 8))
    return -ERR_BAD_ARG;
  if (window < 0 || (window > 0 && !causal)) return -ERR_BAD_ARG;
  if (B <= 0 || S <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  float* delta = reinterpret_cast<float*>(scratch);
  const long delta_bytes = (((long)B * H * S * 4) + 255) & ~255L;
  float* dq_acc = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + delta_bytes);
  const long T = (long)B * S;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, (size_t)T * H * head_dim * 4, st);
  if (e != cudaSuccess) return -(int)e;
  {
    const long threads = T * H * (head_dim / 8);
    attn_delta_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, B, S, H,
                                                                        head_dim, ld_o, ld_do);
  }
  CUtensorMap tq, tk, tv, tdo, tdq;
  int rc;
  if ((rc = make_tmap_tokens_bf16(&tq, q, H * head_dim, S, B, ld_q, 128))) return rc;
  if ((rc = make_tmap_tokens_bf16(&tk, k, Hkv * head_dim, S, B, ld_k, 128))) return rc;
  if ((rc = make_tmap_tokens_bf16(&tv, v, Hkv * head_dim, S, B, ld_v, 128))) return rc;
  if ((rc = make_tmap_tokens_bf16(&tdo, d_o, H * head_dim, S, B, ld_do, 128))) return rc;
  if ((rc = make_tmap_tokens_f32(&tdq, dq_acc, H * head_dim, S, B))) return rc;
  FlashBwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.ld_dk = ld_dk; p.ld_dv = ld_dv;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv; p.scale = scale; p.causal = causal ? 1 : 0; p.window = window >= S ? 0 : window; p.status = status;
  dim3 grid((S + 127) / 128, Hkv, B);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(flash_bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<1>::TOTAL);
    cudaFuncSetAttribute(flash_bwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<2>::TOTAL);
    configured = true;
  }
  if (head_dim == 64) flash_bwd_kernel<1><<<grid, FB_THREADS, BwdSmem<1>::TOTAL, st>>>(tq, tk, tv, tdo, tdq, p);
  else flash_bwd_kernel<2><<<grid, FB_THREADS, BwdSmem<2>::TOTAL, st>>>(tq, tk, tv, tdo, tdq, p);
  {
    const long n = T * H * head_dim / 8;
    long g = (n + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    attn_dq_convert_kernel<<<(unsigned)g, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dq, T, H * head_dim, ld_dq, scale);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

#ifdef FB_TRACE
extern "C" int inv_fb_trace_read(long long* host64) {
  return (int)cudaMemcpyFromSymbol(host64, inv::fb_trace_buf, sizeof(long long) * 64);
}
#endif
