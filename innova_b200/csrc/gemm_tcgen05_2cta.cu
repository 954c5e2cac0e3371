// bf16 GEMM with 2-SM tensor-core instructions (tcgen05.mma.cta_group::2): a pair of CTAs on
// neighbouring SMs computes one 256x256 output tile. Each CTA stages only its own 128 rows of A and
// its own 128 columns of B (32 KB per 64-deep k-block instead of 48 KB for a 128x256 tile), which is
// what lifts the kernel off the shared-memory bandwidth limit that bounds the single-CTA version:
// per k-block a CTA now fills 32 KB and the MMA reads 32 KB, against 48 + 48 KB before.
//
// Protocol inside a pair (cluster of 2, CTA rank 0 is the leader):
//   * both producers TMA-load their halves into their own shared memory; every load signals the
//     LEADER's full barrier (TMA with .cta_group::2, no multicast), which the leader's producer arms
//     with the bytes of both CTAs;
//   * the leader's MMA thread issues the 256x256x16 instructions; the accumulator rows 0-127 live in
//     the leader's TMEM, rows 128-255 in the peer's;
//   * stage release and "accumulator ready" are tcgen05.commit arrivals sent to each CTA's own
//     barrier (two plain commits, one per CTA);
//   * both epilogues drain their TMEM halves and arrive on the leader's tmem_empty barrier.
// Same epilogues, operand layouts (K-major / MN-major) and split-K as the single-CTA kernel.
// Waits are bounded; a cluster barrier at the end keeps both CTAs alive until the pair is done.
#include "gemm_common.cuh"

namespace inv {

namespace g2 {
constexpr int BM = 256, BN = 256, BK = 64, STAGES = 5, UMMA_K = 16;
constexpr int A_STAGE = 128 * BK * 2;  // this CTA's 128 rows of A
constexpr int B_STAGE = 128 * BK * 2;  // this CTA's 128 columns of B
constexpr int THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int STAGING = 8 * 8192;     // per epilogue warp: a 32x64 bf16 box for C and one for the pre-activation
constexpr int SMEM_BYTES = STAGES * (A_STAGE + B_STAGE) + STAGING + 1024 + 384;  // + alignment slack + barriers
constexpr int TMEM_COLS = 512;
}  // namespace g2

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_remote(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
// TMA load whose completion is signalled on a barrier that may live in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (once all MMAs issued so far are complete) on a barrier given by its cluster address.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Output maps of the reduce-scatter form: one per owner rank, over this rank's slot in that owner's receive buffer.
struct RsMaps {
  CUtensorMap m[8];
};

struct WorkUnit2 {
  int m0, n0, kb_begin, kb_end;
  int ag_tile;  // 256-row tile of the gathered operand this unit reads, -1 when it is local or nothing is gathered
};
__device__ __forceinline__ WorkUnit2 decode_work2(int w, const GemmParams& p, int m_tiles, int n_tiles, int kb_total, int kb_per_split) {
  WorkUnit2 u;
  u.ag_tile = -1;
  int n_blk, m_blk, ks;
  if (p.ag_world > 1 && p.ag_operand == 1) {  // B is gathered: all m-tiles of an n-tile before the next n-tile, local shard first
    m_blk = w % m_tiles;
    const int rest = w / m_tiles;
    n_blk = rest % n_tiles;
    ks = rest / n_tiles;
    const int per = p.ag_shard_rows / g2::BN;
    n_blk = (n_blk + p.ag_rank * per) % n_tiles;
    if (n_blk / per != p.ag_rank) u.ag_tile = n_blk;
  } else {
    n_blk = w % n_tiles;
    const int rest = w / n_tiles;
    m_blk = rest % m_tiles;
    ks = rest / m_tiles;
    if (p.ag_world > 1) {  // A is gathered: local rows first, then the peers' in the order the copiers fetch them
      const int per = p.ag_shard_rows / g2::BM;
      m_blk = (m_blk + p.ag_rank * per) % m_tiles;
      if (m_blk / per != p.ag_rank) u.ag_tile = m_blk;
    } else if (p.rs_world > 1) {  // reduce-scatter: the next rank's rows first, the local rows last
      m_blk = (m_blk + (p.rs_rank + 1) * (p.rs_shard_rows / g2::BM)) % m_tiles;
    }
  }
  u.m0 = m_blk * g2::BM;
  u.n0 = n_blk * g2::BN;
  u.kb_begin = ks * kb_per_split;
  u.kb_end = min(kb_total, u.kb_begin + kb_per_split);
  return u;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(g2::THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_aux, const __grid_constant__ RsMaps rs_maps,
                      const GemmParams p) {
  using namespace g2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE;
  uint8_t* sStage = smem + STAGES * (A_STAGE + B_STAGE);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sStage + STAGING);  // used in the leader
  uint64_t* empty_bar = full_bar + STAGES;                                                 // one set per CTA
  uint64_t* tmem_full = empty_bar + STAGES;                                                // one set per CTA
  uint64_t* tmem_empty = tmem_full + 2;                                                    // used in the leader
  uint64_t* aux_bar = tmem_empty + 2;  // two per epilogue warp: "second operand box has landed" (TMA loads of the residual / pre-activation)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_bar + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  // with a fused all-gather the first clusters of the grid only copy; they own no barriers and no tensor memory
  const int n_copy = p.ag_world > 1 ? p.ag_copy_ctas : (p.side.kind != JOB_NONE ? p.side.n_ctas : 0);
  if ((int)blockIdx.x < n_copy) {
    if (p.ag_world > 1) ag_copier(p, 256, smem, full_bar, abort_flag);
    else run_side_job(p.side, (int)blockIdx.x, smem);
    return;
  }
  const int pair = ((int)blockIdx.x - n_copy) >> 1, npairs = ((int)gridDim.x - n_copy) >> 1;

  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_per_split = (kb_total + p.split_k - 1) / p.split_k;
  const int total_work = m_tiles * n_tiles * p.split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // the leader's producer arms it with the bytes of both CTAs
      mbar_init(&empty_bar[s], 1);  // one commit from the leader's MMA thread
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 16);  // 8 epilogue warps in each CTA
    }
    for (int i = 0; i < 16; ++i) mbar_init(&aux_bar[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
    tma_prefetch_desc(&tmap_aux);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int w = pair; ok && w < total_work; w += npairs) {
        const WorkUnit2 u = decode_work2(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
        const int my_m0 = u.m0 + (int)cta * 128;
        const int my_n0 = u.n0 + (int)cta * 128;
        if (u.ag_tile >= 0 && !ag_wait_tile(p, u.ag_tile, abort_flag)) break;
        for (int kb = u.kb_begin; kb < u.kb_end; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t leader_full = mapa_shared(smem_u32(&full_bar[s]), 0);
          // Only the leader arms the barrier, locally and for both CTAs' bytes: a remote arrive would put
          // a cluster-scope release fence on the producer's critical path every stage. The phase cannot
          // complete before that arrival, and the peer cannot run a ring cycle ahead of it because its
          // own empty barrier is released by MMAs that waited on this very phase.
          if (leader) mbar_expect_tx(&full_bar[s], 2 * (A_STAGE + B_STAGE));
          uint8_t* a_dst = sA + s * A_STAGE;
          uint8_t* b_dst = sB + s * B_STAGE;
          const int k0 = kb * BK;
          if (A_MN) {
            tma_load_2d_pair(a_dst, &tmap_a, leader_full, my_m0, k0);
            tma_load_2d_pair(a_dst + 8192, &tmap_a, leader_full, my_m0 + 64, k0);
          } else {
            tma_load_2d_pair(a_dst, &tmap_a, leader_full, k0, my_m0);
          }
          if (B_MN) {
            tma_load_2d_pair(b_dst, &tmap_b, leader_full, my_n0, k0);
            tma_load_2d_pair(b_dst + 8192, &tmap_b, leader_full, my_n0 + 64, k0);
          } else {
            tma_load_2d_pair(b_dst, &tmap_b, leader_full, k0, my_n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only) ----------------
    if (leader && lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      const uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u, sbo = 1024u;
      const uint32_t a_kstep = A_MN ? 2048u : 32u, b_kstep = B_MN ? 2048u : 32u;
      // One thread executes a dependent instruction every few cycles, so everything that can be is hoisted out of the
      // k loop: descriptors and barrier addresses advance by additions, the ring position is a counter.
      const uint64_t da0 = make_smem_desc(smem_u32(sA), a_lbo, sbo, 2), db0 = make_smem_desc(smem_u32(sB), b_lbo, sbo, 2);
      const uint32_t a_k = a_kstep >> 4, b_k = b_kstep >> 4;
      const uint32_t e0 = mapa_shared(smem_u32(&empty_bar[0]), 0), e1 = mapa_shared(smem_u32(&empty_bar[0]), 1);
      int s = 0, tile_i = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int w = pair; ok && w < total_work; w += npairs, ++tile_i) {
        const WorkUnit2 u = decode_work2(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
        const int acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = u.kb_begin; kb < u.kb_end; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = da0 + (uint64_t)(s * (A_STAGE >> 4)), db = db0 + (uint64_t)(s * (B_STAGE >> 4));
          umma_bf16_pair(d_tmem, da, db, idesc, kb > u.kb_begin ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < BK / UMMA_K; ++k) umma_bf16_pair(d_tmem, da + k * a_k, db + k * b_k, idesc, 1u);
          // free this stage in both CTAs
          umma_commit_pair(e0 + s * 8);
          umma_commit_pair(e1 + s * 8);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        const uint32_t f_local = smem_u32(&tmem_full[acc]);
        umma_commit_pair(mapa_shared(f_local, 0));
        umma_commit_pair(mapa_shared(f_local, 1));
      }
    }
  } else {
    // ---------------- epilogue (both CTAs; each drains its own 128 accumulator rows) ----------------
    // 8 warps: warp w reads TMEM lanes 32*(w%4)..+31; warps 2-5 take columns 0-127, warps 6-9 columns 128-255
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const bool staged = !p.c_f32;
    const bool staged_aux = staged && INV_EPI_WRITES_AUX(p.epilogue) && p.aux_out != nullptr;
    // Second operand of the epilogue (residual to add, pre-activation of the GELU backward) through TMA: the warp's two
    // 4 KB boxes alternate; box i is loaded while box i-1 is computed, the result overwrites the operand in place and
    // leaves through a TMA store. Per-thread global loads of a row-strided operand serialise on memory latency
    // (sixteen dependent round trips per tile) and made these epilogues three times as long as the main loop.
    const bool aux_tma = staged && INV_EPI_READS_AUX(p.epilogue);
    uint8_t* my_stage = sStage + (warp - 2) * 8192;
    uint64_t* my_aux_bar = aux_bar + (warp - 2) * 2;
    const int row_in_tile = (int)cta * 128 + q * 32;
    // (w, j): j-th 64-column box of this warp in work unit w; false when the unit or the box does not exist
    auto box_of = [&](int w, int j, int& col0, int& row0) -> bool {
      if (w >= total_work) return false;
      const WorkUnit2 u = decode_work2(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
      col0 = u.n0 + (half * 4 + 2 * j) * 32;
      row0 = u.m0 + row_in_tile;
      return col0 < p.N;
    };
    uint32_t boxes_done = 0;       // boxes this warp has computed: box i uses buffer i & 1, phase (i >> 1) & 1 of its barrier
    int nw = pair, nj = 0;          // next box to prefetch
    auto prefetch_next = [&](uint32_t box_index) {   // lane 0 only
      int col0, row0;
      while (nw < total_work && !box_of(nw, nj, col0, row0)) { nw += npairs; nj = 0; }   // a missing box 0 or 1 ends the unit for this warp
      if (nw >= total_work) return;
      const uint32_t b = box_index & 1;
      mbar_expect_tx(&my_aux_bar[b], 4096);
      tma_load_2d(my_stage + b * 4096, &tmap_aux, &my_aux_bar[b], col0, row0);
      if (nj == 0) nj = 1; else { nj = 0; nw += npairs; }
    };
    if (aux_tma && lane == 0) prefetch_next(0);
    int tile_i = 0;
    bool ok = true;
    for (int w = pair; ok && w < total_work; w += npairs, ++tile_i) {
      const WorkUnit2 u = decode_work2(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
      const int acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (!mbar_wait_warp(&tmem_full[acc], acc_ph, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = u.m0 + row_in_tile + lane;
      const bool row_ok = row < p.M;
      const CUtensorMap* c_map = &tmap_c;
      int row_shift = 0;
      if (p.rs_world > 1) {  // this tile's rows belong to one owner: the staged tile is TMA-stored into its buffer (peer memory) at the shard-relative row
        const int owner = u.m0 / p.rs_shard_rows;
        c_map = &rs_maps.m[owner];
        row_shift = owner * p.rs_shard_rows;
      }
      const uint32_t t_row = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
      const int row0_abs = u.m0 + row_in_tile;
#pragma unroll 1
      for (int c = half * 4; c < half * 4 + 4; c += 2) {
        const int col0 = u.n0 + c * 32;
        if (col0 >= p.N) break;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(t_row + c * 32, r0);
        tmem_ld_32x32(t_row + c * 32 + 32, r1);
        tmem_ld_wait();
        if (aux_tma) {
          const uint32_t b = boxes_done & 1;
          if (lane == 0) {
            tma_store_wait_read();          // the other buffer's store (box i-1) has left shared memory
            prefetch_next(boxes_done + 1);  // ... so box i+1 may land there while box i is computed
          }
          if (!mbar_wait_warp(&my_aux_bar[b], (boxes_done >> 1) & 1, abort_flag, p.status, ERR_WAIT_MISC)) { ok = false; break; }
          uint8_t* sc = my_stage + b * 4096 + lane * 128;
          gemm_epilogue_chunk(p, row, row_ok, col0, r0, sc, nullptr, 0, lane, sc);
          if (col0 + 32 < p.N) gemm_epilogue_chunk(p, row, row_ok, col0 + 32, r1, sc, nullptr, 1, lane, sc);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(c_map, my_stage + b * 4096, col0, row0_abs - row_shift);
            tma_store_commit();
          }
          ++boxes_done;
        } else if (staged) {
          // bf16 output: registers -> swizzled 32x64 box in shared memory -> one TMA store per box
          if (lane == 0) tma_store_wait_read();  // the previous box of this warp has left shared memory
          __syncwarp();
          uint8_t* sc = my_stage + lane * 128;
          uint8_t* sa = staged_aux ? sc + 4096 : nullptr;
          gemm_epilogue_chunk(p, row, row_ok, col0, r0, sc, sa, 0, lane);
          if (col0 + 32 < p.N) gemm_epilogue_chunk(p, row, row_ok, col0 + 32, r1, sc, sa, 1, lane);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(c_map, my_stage, col0, row0_abs - row_shift);
            if (staged_aux) tma_store_2d(&tmap_aux, my_stage + 4096, col0, row0_abs);
            tma_store_commit();
          }
        } else {
          gemm_epilogue_chunk(p, row, row_ok, col0, r0);
          if (col0 + 32 < p.N) gemm_epilogue_chunk(p, row, row_ok, col0 + 32, r1);
        }
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(mapa_shared(smem_u32(&tmem_empty[acc]), 0));
    }
    if (lane == 0) tma_store_wait_all();  // shared memory must outlive the stores that read it
  }

  // ---------------- teardown ----------------
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  tc_fence_before();
  cluster_sync_all();  // neither CTA releases shared memory or TMEM while the other may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
static int launch_gemm_2cta(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx, const RsMaps& rs,
                            const GemmParams& p, int grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_2cta_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, g2::SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  gemm_bf16_2cta_kernel<A_MN, B_MN><<<grid, g2::THREADS, g2::SMEM_BYTES, stream>>>(ta, tb, tc, tx, rs, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// Called by inv_gemm_bf16 when the problem is large enough for 256x256 tiles.
int gemm_2cta_dispatch(const void* A, const void* B, const GemmParams& p0, int lda, int ldb, int a_mn, int b_mn, int num_sms,
                       cudaStream_t stream) {
  using namespace g2;
  GemmParams p = p0;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tmap_2d_bf16(&ta, A, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)lda, 64, BK);
  else rc = make_tmap_2d_bf16(&ta, A, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda, BK, 128);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d_bf16(&tb, B, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)ldb, 64, BK);
  else rc = make_tmap_2d_bf16(&tb, B, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb, BK, 128);
  if (rc) return rc;
  // output maps for the staged TMA-store epilogue (bf16 C and, for the GELU epilogue, the pre-activation)
  CUtensorMap tc = ta, tx = ta;
  if (!p.c_f32) {
    if ((rc = make_tmap_2d_bf16(&tc, p.C, (uint64_t)p.N, (uint64_t)p.M, (uint64_t)p.ldc, 64, 32))) return rc;
    tx = tc;
    if (INV_EPI_WRITES_AUX(p.epilogue) && p.aux_out != nullptr &&
        (rc = make_tmap_2d_bf16(&tx, p.aux_out, (uint64_t)p.N, (uint64_t)p.M, (uint64_t)p.ld_aux, 64, 32)))
      return rc;
    if (INV_EPI_READS_AUX(p.epilogue) &&   // the epilogue's second operand arrives through TMA loads
        (rc = make_tmap_2d_bf16(&tx, p.aux_in, (uint64_t)p.N, (uint64_t)p.M, (uint64_t)p.ld_aux, 64, 32)))
      return rc;
  }
  const int kb_total = (p.K + BK - 1) / BK;
  int split_k = p.split_k < 1 ? 1 : p.split_k;
  if (split_k > kb_total) split_k = kb_total;
  if (p.epilogue != EPI_ATOMIC) split_k = 1;
  {
    const int per = (kb_total + split_k - 1) / split_k;
    split_k = (kb_total + per - 1) / per;
  }
  p.split_k = split_k;
  const long total = (long)((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * split_k;
  // helper CTAs come in whole clusters; the whole grid must be resident at once
  int n_copy = 0;
  if (p.ag_world > 1) {
    n_copy = p.ag_copy_ctas & ~1;
    p.side.kind = JOB_NONE;
  } else if (p.side.kind != JOB_NONE) {
    n_copy = p.side.n_ctas & ~1;
    if (n_copy < 2) n_copy = 2;
    p.side.n_ctas = n_copy;
  }
  p.ag_copy_ctas = p.ag_world > 1 ? n_copy : 0;
  const int max_pairs = (num_sms - n_copy) / 2;
  const int pairs = (int)(total < max_pairs ? total : max_pairs);
  const int grid = pairs * 2 + n_copy;
  RsMaps rs;
  for (int r = 0; r < 8; ++r) rs.m[r] = tc;
  if (p.rs_world > 1 && !p.c_f32) {
    for (int r = 0; r < p.rs_world; ++r)
      if ((rc = make_tmap_2d_bf16(&rs.m[r], p.rs_dst[r], (uint64_t)p.N, (uint64_t)p.rs_shard_rows, (uint64_t)p.ldc, 64, 32))) return rc;
  }
  if (a_mn && b_mn) return launch_gemm_2cta<true, true>(ta, tb, tc, tx, rs, p, grid, stream);
  if (a_mn && !b_mn) return launch_gemm_2cta<true, false>(ta, tb, tc, tx, rs, p, grid, stream);
  if (!a_mn && b_mn) return launch_gemm_2cta<false, true>(ta, tb, tc, tx, rs, p, grid, stream);
  return launch_gemm_2cta<false, false>(ta, tb, tc, tx, rs, p, grid, stream);
}

}  // namespace inv
