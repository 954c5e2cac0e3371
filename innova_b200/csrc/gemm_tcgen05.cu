// bf16 GEMM on 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T with fused epilogues.
//
// Replaces the reference's CPU GEMMs (src/kernel_gemm.cpp:13-118, src/math_avx2_tiled.cpp:308-527:
// GEMM + bias + activation) and its 16x16 shader GEMM (src/gpu_compute_full.cpp:29-69).
//
// Design (one persistent CTA per SM, 320 threads, warp-specialised):
//   warp 0   : TMA producer. Streams 128x64 A tiles and 256x64 B tiles into a 4-stage ring of
//              128B-swizzled shared memory.
//   warp 1   : allocates all 512 TMEM columns and issues tcgen05.mma (M=128, N=256, K=16) from one
//              thread. Two 128x256 fp32 accumulators live in TMEM, so that the mainloop of tile i+1
//              overlaps the epilogue of tile i.
//   warps 2-9: epilogue. tcgen05.ld the accumulator (one row per thread), apply bias / GELU /
//              GELU-backward / residual add, and store bf16 or fp32; a split-K unit instead adds
//              its partial sums into an fp32 C with vector reductions.
// Either operand may be K-major ([rows, K] row-major) or MN-major ([K, rows] row-major); the latter
// lets the backward GEMMs (dgrad reads W[N,K] along N, wgrad reads X and dY along tokens) run with no
// transposes in memory.
// All waits are bounded; a wait that runs out writes a code into *status and the CTA unwinds.
#include "gemm_common.cuh"

#include <mutex>

namespace inv {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int GEMM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int GEMM_SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 512;


struct WorkUnit {
  int m0, n0, kb_begin, kb_end;
  int b_row_off;   // extra row offset into the stacked B (grouped mode 1)
  int bias_off;
  long c_off;      // element offset of this unit's C (grouped mode 2)
  bool skip;
  int ag_tile;     // tile index of the gathered operand this unit reads, -1 when it is local or nothing is gathered
};
__device__ __forceinline__ WorkUnit decode_work(int w, const GemmParams& p, int m_tiles, int n_tiles, int kb_total, int kb_per_split) {
  WorkUnit u;
  u.b_row_off = 0;
  u.bias_off = 0;
  u.c_off = 0;
  u.skip = false;
  u.ag_tile = -1;
  int n_blk, m_blk, rest;
  if (p.ag_world > 1 && p.ag_operand == 1) {  // B is gathered: walk all m-tiles of an n-tile before the next n-tile
    m_blk = w % m_tiles;
    rest = w / m_tiles;
    n_blk = rest % n_tiles;
    rest /= n_tiles;
    const int per = p.ag_shard_rows / BN;
    n_blk = (n_blk + p.ag_rank * per) % n_tiles;
    if (n_blk / per != p.ag_rank) u.ag_tile = n_blk;
  } else {
    n_blk = w % n_tiles;
    rest = w / n_tiles;
    m_blk = rest % m_tiles;
    rest /= m_tiles;
    if (p.ag_world > 1) {
      const int per = p.ag_shard_rows / BM;
      m_blk = (m_blk + p.ag_rank * per) % m_tiles;
      if (m_blk / per != p.ag_rank) u.ag_tile = m_blk;
    } else if (p.rs_world > 1) {
      m_blk = (m_blk + (p.rs_rank + 1) * (p.rs_shard_rows / BM)) % m_tiles;
    }
  }
  u.m0 = m_blk * BM;
  u.n0 = n_blk * BN;
  if (p.group_mode == 2) {
    const int ks = rest % p.split_k, e = rest / p.split_k;
    const int off = p.group_offsets[e], len = p.group_offsets[e + 1] - off;
    const int nkb = len / BK, per = (nkb + p.split_k - 1) / p.split_k;
    u.kb_begin = off / BK + ks * per;
    u.kb_end = min(off / BK + nkb, u.kb_begin + per);
    u.c_off = (long)e * p.group_stride_c;
    u.skip = u.kb_begin >= u.kb_end;
    return u;
  }
  const int ks = rest;
  u.kb_begin = ks * kb_per_split;
  u.kb_end = min(kb_total, u.kb_begin + kb_per_split);
  if (p.group_mode == 1) {
    const int e = p.tile_expert[m_blk];
    u.skip = e < 0;
    u.b_row_off = e < 0 ? 0 : e * p.group_rows_b;
    u.bias_off = e < 0 ? 0 : e * p.group_stride_bias;
  }
  return u;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // with a fused all-gather the first CTAs of the grid only copy; they own no barriers and no TMEM
  const int n_copy = p.ag_world > 1 ? p.ag_copy_ctas : 0;
  if ((int)blockIdx.x < n_copy) {
    ag_copier(p, p.ag_operand == 1 ? BN : BM, smem, full_bar, abort_flag);
    return;
  }
  const int bid = blockIdx.x - n_copy, gdim = gridDim.x - n_copy;

  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_per_split = (kb_total + p.split_k - 1) / p.split_k;
  const int total_work = m_tiles * n_tiles * p.split_k * (p.group_mode == 2 ? p.num_groups : 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
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
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;
      for (int w = bid; w < total_work; w += gdim) {
        WorkUnit u = decode_work(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
        if (u.skip) continue;
        bool ok = true;
        if (u.ag_tile >= 0 && !ag_wait_tile(p, u.ag_tile, abort_flag)) break;
        for (int kb = u.kb_begin; kb < u.kb_end; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full_bar[s], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmap_a, &full_bar[s], u.m0 + j * 64, k0);
          } else {
            tma_load_2d(a_dst, &tmap_a, &full_bar[s], k0, u.m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmap_b, &full_bar[s], u.n0 + j * 64, k0 + u.b_row_off);
          } else {
            tma_load_2d(b_dst, &tmap_b, &full_bar[s], k0, u.n0 + u.b_row_off);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      // K-major, 128B swizzle: 8-row groups are 1024 B apart. MN-major (64-wide boxes of BK rows):
      // 64-element groups along MN are one box (8192 B) apart, 8-row groups along K 1024 B apart.
      uint32_t a_lbo = A_MN ? 8192u : 16u, a_sbo = 1024u;
      uint32_t b_lbo = B_MN ? 8192u : 16u, b_sbo = 1024u;
      const uint32_t a_kstep = A_MN ? 2048u : 32u;
      const uint32_t b_kstep = B_MN ? 2048u : 32u;
      // One thread executes a dependent instruction every few cycles, so everything that can be is hoisted out of the
      // k loop: descriptors advance by additions, the ring position is a counter.
      const uint64_t da0 = make_smem_desc(smem_u32(sA), a_lbo, a_sbo, 2), db0 = make_smem_desc(smem_u32(sB), b_lbo, b_sbo, 2);
      const uint32_t a_k = a_kstep >> 4, b_k = b_kstep >> 4;
      int s = 0, tile_i = 0;
      uint32_t ph = 0;
      for (int w = bid; w < total_work; w += gdim) {
        WorkUnit u = decode_work(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
        if (u.skip) continue;
        const int acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = u.kb_begin; kb < u.kb_end; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = da0 + (uint64_t)(s * (A_STAGE_BYTES >> 4)), db = db0 + (uint64_t)(s * (B_STAGE_BYTES >> 4));
          umma_bf16(d_tmem, da, db, idesc, kb > u.kb_begin ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < BK / UMMA_K; ++k) umma_bf16(d_tmem, da + k * a_k, db + k * b_k, idesc, 1u);
          umma_commit(&empty_bar[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        ++tile_i;
      }
    }
  } else {
    // ---------------- epilogue (4 warps; warp w may touch TMEM lanes 32*(w%4)..+31) ----------------
    // 8 warps: warp w reads TMEM lanes 32*(w%4)..+31; warps 2-5 take columns 0-127, warps 6-9 columns 128-255
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int tile_i = 0;
    for (int w = bid; w < total_work; w += gdim) {
      WorkUnit u = decode_work(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
      if (u.skip) continue;
      GemmParams pe = p;  // this unit's view of the outputs (grouped modes shift bias / C)
      if (p.group_mode) {
        if (pe.bias) pe.bias += u.bias_off;
        pe.C = p.c_f32 ? (void*)(reinterpret_cast<float*>(p.C) + u.c_off) : (void*)(reinterpret_cast<__nv_bfloat16*>(p.C) + u.c_off);
      }
      const int acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (!mbar_wait_warp(&tmem_full[acc], acc_ph, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      int row = u.m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      if (p.rs_world > 1) {  // this tile's rows belong to one owner: add into its buffer at the shard-relative row
        const int owner = u.m0 / p.rs_shard_rows;
        pe.C = p.rs_dst[owner];
        row -= owner * p.rs_shard_rows;
      }
      const uint32_t t_row = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
#pragma unroll 1
      for (int c = half * 4; c < half * 4 + 4; c += 2) {
        const int col0 = u.n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(t_row + c * 32, r0);
        tmem_ld_32x32(t_row + c * 32 + 32, r1);
        tmem_ld_wait();
        gemm_epilogue_chunk(pe, row, row_ok, col0, r0);
        if (col0 + 32 < p.N) gemm_epilogue_chunk(pe, row, row_ok, col0 + 32, r1);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      ++tile_i;
    }
  }

  // ---------------- teardown ----------------
  __syncthreads();
  if (*abort_flag) {
    // Give copies and MMAs still in flight a bounded time to land before TMEM is released.
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
// Host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows of `ld` elements; 128B swizzle.
int make_tmap_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                      uint32_t box_outer) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

template <bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  gemm_bf16_kernel<A_MN, B_MN><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

static int g_num_sms = 0;

int gemm_2cta_dispatch(const void* A, const void* B, const GemmParams& p0, int lda, int ldb, int a_mn, int b_mn, int num_sms,
                       cudaStream_t stream);

}  // namespace inv

using namespace inv;

static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                         int b_mn, int epilogue, const void* bias, const void* aux_in, int ld_aux, void* aux_out, int c_f32,
                         int split_k, float alpha, int* status, void* stream, int kernel_select, const SideJob* job) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // TMA needs 16-byte aligned bases and row pitches; the vector epilogue needs N % 8 == 0.
  if ((lda % 8) || (ldb % 8) || (ldc % (c_f32 ? 4 : 8)) || (N % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15))
    return -ERR_BAD_ARG;
  if (epilogue == EPI_ATOMIC && !c_f32) return -ERR_BAD_ARG;
  if (INV_EPI_READS_AUX(epilogue) && (aux_in == nullptr || (ld_aux % 8))) return -ERR_BAD_ARG;
  if (epilogue == EPI_GELU_DG && (aux_out == nullptr || (ld_aux % 8))) return -ERR_BAD_ARG;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  if (job != nullptr && !(kernel_select != 1 && M > 128 && N > 128)) return -ERR_BAD_ARG;  // only the CTA-pair kernel carries side jobs
  if (kernel_select != 1 && M > 128 && N > 128) {
    // large problems: 256x256 tiles on CTA pairs (gemm_tcgen05_2cta.cu)
    GemmParams q;
    q.M = M; q.N = N; q.K = K; q.split_k = split_k;
    q.C = C; q.ldc = ldc; q.c_f32 = c_f32;
    q.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
    q.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_in);
    q.ld_aux = ld_aux;
    q.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
    q.epilogue = epilogue;
    q.alpha = alpha;
    q.status = status;
    q.group_mode = 0; q.num_groups = 1; q.tile_expert = nullptr; q.group_offsets = nullptr; q.group_rows_b = 0;
    q.group_stride_bias = 0; q.group_stride_c = 0;
    if (job != nullptr) q.side = *job;
    return gemm_2cta_dispatch(A, B, q, lda, ldb, a_mn, b_mn, g_num_sms, reinterpret_cast<cudaStream_t>(stream));
  }
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK);
  else rc = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK);
  else rc = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN);
  if (rc) return rc;

  const int kb_total = (K + BK - 1) / BK;
  if (split_k < 1) split_k = 1;
  if (split_k > kb_total) split_k = kb_total;
  if (epilogue != EPI_ATOMIC) split_k = 1;
  {  // no empty split may exist
    int per = (kb_total + split_k - 1) / split_k;
    split_k = (kb_total + per - 1) / per;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.split_k = split_k;
  p.C = C; p.ldc = ldc; p.c_f32 = c_f32;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_in);
  p.ld_aux = ld_aux;
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
  p.epilogue = epilogue;
  p.alpha = alpha;
  p.status = status;
  p.group_mode = 0; p.num_groups = 1; p.tile_expert = nullptr; p.group_offsets = nullptr; p.group_rows_b = 0;
  p.group_stride_bias = 0; p.group_stride_c = 0;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const long total = (long)m_tiles * n_tiles * split_k;
  int grid = (int)(total < g_num_sms ? total : g_num_sms);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn && b_mn) return launch_gemm<true, true>(ta, tb, p, grid, st);
  if (a_mn && !b_mn) return launch_gemm<true, false>(ta, tb, p, grid, st);
  if (!a_mn && b_mn) return launch_gemm<false, true>(ta, tb, p, grid, st);
  return launch_gemm<false, false>(ta, tb, p, grid, st);
}


extern "C" int inv_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                             int b_mn, int epilogue, const void* bias, const void* aux_in, int ld_aux, void* aux_out, int c_f32,
                             int split_k, float alpha, int* status, void* stream, int kernel_select) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epilogue, bias, aux_in, ld_aux, aux_out, c_f32, split_k, alpha, status,
                        stream, kernel_select, nullptr);
}

// The same GEMM with a side job (side_job.cuh) run by the first job->n_ctas CTAs of its grid. Only problems that take
// the CTA-pair kernel (M > 128 and N > 128) can carry one; others are refused.
extern "C" int inv_gemm_bf16_job(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                                 int b_mn, int epilogue, const void* bias, const void* aux_in, int ld_aux, void* aux_out, int c_f32,
                                 int split_k, float alpha, int* status, void* stream, const void* job) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epilogue, bias, aux_in, ld_aux, aux_out, c_f32, split_k, alpha, status,
                        stream, 0, reinterpret_cast<const SideJob*>(job));
}

static void fill_plain(GemmParams& p, int M, int N, int K, void* C, int ldc, int c_f32, const void* bias, const void* aux_in, int ld_aux,
                       void* aux_out, int epilogue, float alpha, int* status) {
  p.M = M; p.N = N; p.K = K; p.split_k = 1;
  p.C = C; p.ldc = ldc; p.c_f32 = c_f32;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_in);
  p.ld_aux = ld_aux;
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
  p.epilogue = epilogue; p.alpha = alpha; p.status = status;
  p.group_mode = 0; p.num_groups = 1; p.tile_expert = nullptr; p.group_offsets = nullptr; p.group_rows_b = 0;
  p.group_stride_bias = 0; p.group_stride_c = 0;
}

// All-gather fused into a GEMM: C[M, N] = A[M, K] * B[N, K]^T where the gathered operand (operand 0: A, 1: B)
// is sharded by rows over W ranks. `peer_bufs[r]` is rank r's full-size buffer of that operand ([W * shard_rows, ld]
// bf16) which holds at least rank r's own shard; this rank's buffer is peer_bufs[rank] and receives the other
// shards. flags: >= (W * shard_rows / tile) device words on this GPU, epoch: a value not used on them before.
// All ranks must have written their shard before the launch and must not overwrite it before every rank's
// kernel has finished (the caller brackets the call with barriers).
extern "C" int inv_gemm_ag_bf16(const uint64_t* peer_bufs, int W, int rank, int operand, int shard_rows, int ld_gathered, const void* other,
                                int ld_other, void* C, int ldc, int M, int N, int K, int epilogue, const void* bias, const void* aux_in,
                                int ld_aux, void* aux_out, int c_f32, uint32_t* flags, uint32_t epoch, int copy_ctas, int* status,
                                void* stream) {
  if (W < 1 || W > 8 || rank < 0 || rank >= W || (operand != 0 && operand != 1)) return -ERR_BAD_ARG;
  const int tile_rows = operand ? BN : BM;
  if (shard_rows % tile_rows || (operand ? N : M) != W * shard_rows) return -ERR_BAD_ARG;
  if ((ld_gathered % 8) || (ld_other % 8) || (ldc % (c_f32 ? 4 : 8)) || (N % 8) || (K % 8)) return -ERR_BAD_ARG;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  GemmParams p;
  fill_plain(p, M, N, K, C, ldc, c_f32, bias, aux_in, ld_aux, aux_out, epilogue, 1.0f, status);
  if (epilogue == EPI_ATOMIC) return -ERR_BAD_ARG;
  void* local = reinterpret_cast<void*>(peer_bufs[rank]);
  const void* A = operand ? other : local;
  const void* B = operand ? local : other;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)(operand ? ld_other : ld_gathered), BK, BM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)(operand ? ld_gathered : ld_other), BK, BN))) return rc;
  p.ag_world = W; p.ag_rank = rank; p.ag_operand = operand; p.ag_shard_rows = shard_rows; p.ag_ld = ld_gathered;
  for (int r = 0; r < W; ++r) p.ag_src[r] = reinterpret_cast<const void*>(peer_bufs[r]);
  p.ag_dst = local; p.ag_flags = flags; p.ag_epoch = epoch;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const long total = (long)m_tiles * n_tiles;
  // a copier CTA keeps ~130 KB in flight, i.e. ~40 GB/s over a microseconds-long round trip: enough CTAs to fill the links
  if (W == 1) copy_ctas = 0;
  else if (copy_ctas < 1) copy_ctas = W >= 8 ? 20 : (W >= 4 ? 12 : 8);
  if (copy_ctas > g_num_sms / 4) copy_ctas = g_num_sms / 4;
  p.ag_copy_ctas = copy_ctas;
  // 256x256 tiles on CTA pairs when the shards are whole 256-row tiles (the faster kernel)
  if (shard_rows % 256 == 0 && M >= 512 && N >= 256 && K % 64 == 0)
    return gemm_2cta_dispatch(A, B, p, operand ? ld_other : ld_gathered, operand ? ld_gathered : ld_other, 0, 0, g_num_sms,
                              reinterpret_cast<cudaStream_t>(stream));
  long gemm_ctas = total < g_num_sms - copy_ctas ? total : g_num_sms - copy_ctas;
  // the whole grid must be resident at once (the GEMM CTAs wait for the copier CTAs): one CTA per SM
  return launch_gemm<false, false>(ta, tb, p, (int)gemm_ctas + copy_ctas, reinterpret_cast<cudaStream_t>(stream));
}

// GEMM fused with a reduce-scatter: every rank computes the full [M, N] partial product of its K-slice and adds
// row shard r (M / W rows) into rank r's fp32 buffer peer_out[r] ([M / W, ldc]), which must be zero (or hold a
// value to add to) before any rank starts.
extern "C" int inv_gemm_rs_bf16(const void* A, int lda, const void* B, int ldb, const uint64_t* peer_out, int W, int rank, int ldc, int M,
                                int N, int K, float alpha, int* status, void* stream) {
  if (W < 1 || W > 8 || rank < 0 || rank >= W || M % W || (M / W) % BM) return -ERR_BAD_ARG;
  if ((lda % 8) || (ldb % 8) || (ldc % 4) || (N % 8)) return -ERR_BAD_ARG;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  GemmParams p;
  fill_plain(p, M, N, K, reinterpret_cast<void*>(peer_out[rank]), ldc, 1, nullptr, nullptr, 0, nullptr, EPI_ATOMIC, alpha, status);
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN))) return rc;
  p.rs_world = W; p.rs_rank = rank; p.rs_shard_rows = M / W;
  for (int r = 0; r < W; ++r) p.rs_dst[r] = reinterpret_cast<float*>(peer_out[r]);
  const long total = (long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return launch_gemm<false, false>(ta, tb, p, (int)(total < g_num_sms ? total : g_num_sms), reinterpret_cast<cudaStream_t>(stream));
}


// Grouped GEMM over expert segments (see GemmParams::group_mode), always on the single-CTA kernel.
//   mode 1: C[R, N] = A[R, K] * B_e^T per 128-row tile, e = tile_expert[tile]; B stacked [E * rows_b, ...].
//           M = R is the static row capacity of the permuted buffer.
//   mode 2: C_e[M, N] += sum over the rows of group e (A: [R, M] a_mn, B: [R, N] b_mn), fp32 atomics.
extern "C" int inv_gemm_grouped(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn,
                                int epilogue, const void* bias, const void* aux_in, int ld_aux, void* aux_out, int c_f32, int split_k,
                                int group_mode, int num_groups, const int* tile_expert, const int* group_offsets, int group_rows_b,
                                int group_stride_bias, long group_stride_c, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (c_f32 ? 4 : 8)) || (N % 8)) return -ERR_BAD_ARG;
  if (group_mode == 2 && (!a_mn || !b_mn || !c_f32 || epilogue != EPI_ATOMIC)) return -ERR_BAD_ARG;
  if (group_mode == 1 && a_mn) return -ERR_BAD_ARG;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  CUtensorMap ta, tb;
  int rc;
  // the stacked B is addressed through one map: its outer extent covers all groups
  const uint64_t b_rows_total = (uint64_t)group_rows_b * (group_mode == 1 ? num_groups : 1);
  if (a_mn) rc = make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK);
  else rc = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d_bf16(&tb, B, (uint64_t)N, group_mode == 1 ? b_rows_total : (uint64_t)K, (uint64_t)ldb, 64, BK);
  else rc = make_tmap_2d_bf16(&tb, B, (uint64_t)K, group_mode == 1 ? b_rows_total : (uint64_t)N, (uint64_t)ldb, BK, BN);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.split_k = group_mode == 2 ? (split_k < 1 ? 1 : split_k) : 1;
  p.C = C; p.ldc = ldc; p.c_f32 = c_f32;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_in);
  p.ld_aux = ld_aux;
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
  p.epilogue = epilogue;
  p.alpha = 1.0f;
  p.status = status;
 
  p.group_mode = group_mode; p.num_groups = num_groups; p.tile_expert = tile_expert; p.group_offsets = group_offsets;
  p.group_rows_b = group_rows_b; p.group_stride_bias = group_stride_bias; p.group_stride_c = group_stride_c;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const long total = (long)m_tiles * n_tiles * p.split_k * (group_mode == 2 ? num_groups : 1);
  const int grid = (int)(total < g_num_sms ? total : g_num_sms);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn && b_mn) return launch_gemm<true, true>(ta, tb, p, grid, st);
  if (!a_mn && b_mn) return launch_gemm<false, true>(ta, tb, p, grid, st);
  if (a_mn && !b_mn) return launch_gemm<true, false>(ta, tb, p, grid, st);
  return launch_gemm<false, false>(ta, tb, p, grid, st);
}

// GEMM fused with a reduce-scatter, push form: every rank computes the full [M, N] partial product of its K-slice in
// bf16 and its epilogue stores the tile rows owned by rank r straight into this rank's slot of r's receive buffer
// (peer_slots[r], [M / W, ldc] bf16, plain 16-byte stores: posted writes over NVLink, no atomics), visiting the
// owners starting after the local rank so that the local rows, which cross no link, come last. The owner then adds
// its W slots (inv_sum_slots_bf16) once every rank has passed a barrier. The transfer overlaps the math tile by tile;
// the bytes on the links are the bf16 partial sums, as in a library reduce-scatter.
extern "C" int inv_gemm_rs_push_bf16(const void* A, int lda, const void* B, int ldb, const uint64_t* peer_slots, int W, int rank, int ldc, int M,
                                     int N, int K, int* status, void* stream) {
  if (W < 1 || W > 8 || rank < 0 || rank >= W || M % W || (M / W) % BM) return -ERR_BAD_ARG;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8)) return -ERR_BAD_ARG;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  GemmParams p;
  fill_plain(p, M, N, K, reinterpret_cast<void*>(peer_slots[rank]), ldc, 0, nullptr, nullptr, 0, nullptr, EPI_NONE, 1.0f, status);
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN))) return rc;
  p.rs_world = W; p.rs_rank = rank; p.rs_shard_rows = M / W;
  for (int r = 0; r < W; ++r) p.rs_dst[r] = reinterpret_cast<float*>(peer_slots[r]);  // typed by c_f32 in the epilogue
  if ((M / W) % 256 == 0 && N >= 256 && K % 64 == 0)
    return gemm_2cta_dispatch(A, B, p, lda, ldb, 0, 0, g_num_sms, reinterpret_cast<cudaStream_t>(stream));
  const long total = (long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return launch_gemm<false, false>(ta, tb, p, (int)(total < g_num_sms ? total : g_num_sms), reinterpret_cast<cudaStream_t>(stream));
}

namespace inv {
// out[i] = bf16(sum_w slots[w * stride + i]), eight elements per thread.
__global__ void sum_slots_bf16_kernel(const __nv_bfloat16* __restrict__ slots, long stride, int W, __nv_bfloat16* __restrict__ out, long n8) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < W; ++w) {
      const uint4 v = *reinterpret_cast<const uint4*>(slots + w * stride + i * 8);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(u[j] << 16);
        acc[2 * j + 1] += __uint_as_float(u[j] & 0xffff0000u);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]); o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }
}
}  // namespace inv

extern "C" int inv_sum_slots_bf16(const void* slots, long stride_elems, int W, void* out, long n, void* stream) {
  if (n % 8 || stride_elems % 8) return -ERR_BAD_ARG;
  const long n8 = n / 8;
  long grid = (n8 + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  inv::sum_slots_bf16_kernel<<<(int)grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)slots, stride_elems, W, (__nv_bfloat16*)out, n8);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
