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
};
__device__ __forceinline__ WorkUnit decode_work(int w, const GemmParams& p, int m_tiles, int n_tiles, int kb_total, int kb_per_split) {
  WorkUnit u;
  u.b_row_off = 0;
  u.bias_off = 0;
  u.c_off = 0;
  u.skip = false;
  const int n_blk = w % n_tiles;
  int rest = w / n_tiles;
  const int m_blk = rest % m_tiles;
  rest /= m_tiles;
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
      for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
        WorkUnit u = decode_work(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
        if (u.skip) continue;
        bool ok = true;
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
      if (p.swap_lbo_sbo) {
        if (A_MN) { uint32_t t = a_lbo; a_lbo = a_sbo; a_sbo = t; }
        if (B_MN) { uint32_t t = b_lbo; b_lbo = b_sbo; b_sbo = t; }
      }
      const uint32_t a_kstep = A_MN ? 2048u : 32u;
      const uint32_t b_kstep = B_MN ? 2048u : 32u;
      int it = 0, tile_i = 0;
      for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
        WorkUnit u = decode_work(w, p, m_tiles, n_tiles, kb_total, kb_per_split);
        if (u.skip) continue;
        const int acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = u.kb_begin; kb < u.kb_end; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc(a_base + k * a_kstep, a_lbo, a_sbo, 2);
            const uint64_t db = make_smem_desc(b_base + k * b_kstep, b_lbo, b_sbo, 2);
            umma_bf16(d_tmem, da, db, idesc, (kb > u.kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
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
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
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
      const int row = u.m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
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

extern "C" int inv_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn,
                             int b_mn, int epilogue, const void* bias, const void* aux_in, int ld_aux, void* aux_out, int c_f32,
                             int split_k, float alpha, int* status, void* stream, int debug_flags) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // TMA needs 16-byte aligned bases and row pitches; the vector epilogue needs N % 8 == 0.
  if ((lda % 8) || (ldb % 8) || (ldc % (c_f32 ? 4 : 8)) || (N % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15))
    return -ERR_BAD_ARG;
  if (epilogue == EPI_ATOMIC && !c_f32) return -ERR_BAD_ARG;
  if ((epilogue == EPI_DGELU || epilogue == EPI_ADD) && (aux_in == nullptr || (ld_aux % 8))) return -ERR_BAD_ARG;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  if (!(debug_flags & 2) && M > 128 && N > 128) {
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
    q.swap_lbo_sbo = debug_flags;
    q.group_mode = 0; q.num_groups = 1; q.tile_expert = nullptr; q.group_offsets = nullptr; q.group_rows_b = 0;
    q.group_stride_bias = 0; q.group_stride_c = 0;
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
  p.swap_lbo_sbo = debug_flags & 1;
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
  p.swap_lbo_sbo = 0;
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
