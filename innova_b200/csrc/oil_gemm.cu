// Weight-only quantised GEMM for OIL4 / OIL8 weights: y[M, N] += x[M, K] * dequant(W)[N, K]^T, with
// the codebook indices expanded inside the kernel on the way from shared memory to the tensor core.
//
// Replaces the reference's gather-FMA kernels oil4_gemm / oil8_gemm (src/kernel_oil4.cpp:31-128,
// src/kernel_oil8.cpp:14-79), the engines' quant_gemm (src/oil_engines_core.cpp:51-160) and the
// production GEMVs gemv_oil4_* / gemv_oil8_* (src/kernel_production.cpp:95-166).
//
// Weight format (the block-32 compute format of csrc/quant.cu): index [N, K] (OIL8: one byte, OIL4:
// two per byte, low nibble first; 2-bit: four per byte, low bits first), scale bf16 [N, K/32], one shared
// codebook over [-1, 1]. The 2-bit path serves the ternary weights (SPARK, OIL1: codebook {-1, 0, +1, 0})
// and OIL2 (four levels) and replaces tl1/tl2_gemm and gemv_spark_* (src/kernel_tl.cpp:32-185,
// src/kernel_production.cpp:79-93).
//
// The kernel is built for the decode shape (M = tokens in flight <= 256, N and K large) and runs
// "swapped": the 128 weight rows of a tile are the M side of tcgen05.mma, the tokens its N side.
//   warp 0    TMA: raw index tiles (128 rows x 64 k) and activation tiles (M x 64 k, 128B swizzle)
//   warp 1    MMA issuer, accumulator [128 weight rows x M tokens] fp32 in TMEM
//   warps 2-9 dequantise: each thread owns one scale block (row, 32 k): reads 16 or 32 index bytes,
//             looks the values up in a shared-memory table of bf16 pairs (OIL4: indexed by the byte,
//             i.e. two weights per lookup), multiplies by the block scale with packed bf16 math and
//             writes its 64 bytes into the swizzled A-operand tile. The same warps run the epilogue.
// With `multimem` set the output pointer is an NVLS multicast address and the epilogue's reductions are
// multimem.red: the switch adds each partial sum into every rank's copy of the buffer, which turns a
// row-parallel (tensor-parallel) linear layer into GEMM + all-reduce in one kernel.
// Small N leaves most SMs idle, so the reduction dimension is split across CTAs (split-K) and the
// partial sums are added to an fp32 output with reductions. Every wait is bounded.
#include "sm100_common.cuh"
#include "inv_api.h"

#include <mutex>

namespace inv {

int make_tmap_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                      uint32_t box_outer);

namespace og {
constexpr int BN = 128;     // weight rows per tile (MMA M)
constexpr int BK = 64;
constexpr int IDX_STAGES = 6, AB_STAGES = 3;
constexpr int THREADS = 320;
constexpr int MAXM = 256;   // tokens per launch (MMA N)
constexpr int A_TILE = BN * BK * 2;  // 16 KB dequantised weights
}  // namespace og

struct OilGemmParams {
  int M, N, K, bits;  // bits = 4 or 8
  int Mpad;           // M rounded up to 16
  const __nv_bfloat16* scales;
  const float* codebook;
  float* out;  // [M, N] fp32
  int ldo;
  int split_k;
  int* status;
  int multimem;  // out is an NVLS multicast address: every partial sum is added into all ranks' copies
};

typedef CUresult (*EncodeTiledFnO)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFnO og_encode_fn() {
  static EncodeTiledFnO fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnO>(f);
  });
  return fn;
}
// Plain (unswizzled) byte tensor map: `inner` bytes per row, `outer` rows.
static int make_tmap_bytes(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFnO enc = og_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

template <int BITS>
__global__ void __launch_bounds__(og::THREADS, 1)
oil_gemm_kernel(const __grid_constant__ CUtensorMap tmap_idx, const __grid_constant__ CUtensorMap tmap_x, const OilGemmParams p) {
  using namespace og;
  constexpr int IDX_TILE = BN * BK * BITS / 8;  // 4 KB (OIL4) or 8 KB (OIL8)
  constexpr int ROW_BYTES = BK * BITS / 8;      // 32 or 64
  const int X_TILE = p.Mpad * BK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                                  // AB_STAGES x 16 KB
  uint8_t* sX = sA + AB_STAGES * A_TILE;               // AB_STAGES x 32 KB (sized for MAXM)
  uint8_t* sIdx = sX + AB_STAGES * (MAXM * BK * 2);    // IDX_STAGES x IDX_TILE
  uint32_t* lut = reinterpret_cast<uint32_t*>(sIdx + IDX_STAGES * IDX_TILE);  // 256 entries x 32 bank copies
  uint64_t* bars = reinterpret_cast<uint64_t*>(lut + 256 * 32);
  uint64_t* idx_full = bars;
  uint64_t* idx_empty = idx_full + IDX_STAGES;
  uint64_t* a_full = idx_empty + IDX_STAGES;
  uint64_t* a_empty = a_full + AB_STAGES;
  uint64_t* x_full = a_empty + AB_STAGES;
  uint64_t* acc_full = x_full + AB_STAGES;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int kb_total = p.K / BK;
  const int kb_per = (kb_total + p.split_k - 1) / p.split_k;
  const int total_work = n_tiles * p.split_k;

  // lookup table: OIL4 -> bf16 pair (codebook[low nibble], codebook[high nibble]) per byte; OIL8 -> one bf16
  // entry e for lane l lives at lut[e * 32 + l]: every lane reads its own bank, whatever the indices are
  for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
    const int e = i >> 5;
    if (BITS == 2) lut[i] = 0;
    else if (BITS == 4) lut[i] = pack_bf16x2(p.codebook[e & 15], p.codebook[e >> 4]);
    else lut[i] = pack_bf16x2(p.codebook[e], 0.f);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < IDX_STAGES; ++s) {
      mbar_init(&idx_full[s], 1);
      mbar_init(&idx_empty[s], 256);
    }
    for (int s = 0; s < AB_STAGES; ++s) {
      mbar_init(&a_full[s], 256);
      mbar_init(&a_empty[s], 1);
      mbar_init(&x_full[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 256);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_idx);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // lane 0 streams index tiles, lane 1 streams activation tiles; each runs ahead on its own ring
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const int n0 = (w % n_tiles) * BN;
        const int kb0 = (w / n_tiles) * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int si = it % IDX_STAGES;
          if (!mbar_wait(&idx_empty[si], ((it / IDX_STAGES) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&idx_full[si], IDX_TILE);
          tma_load_2d(sIdx + si * IDX_TILE, &tmap_idx, &idx_full[si], kb * ROW_BYTES, n0);
        }
      }
    } else if (lane == 1) {
      int it = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const int kb0 = (w / n_tiles) * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int sx = it % AB_STAGES;
          // the x stage is released together with the A stage (same MMA commit)
          if (!mbar_wait(&a_empty[sx], ((it / AB_STAGES) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&x_full[sx], X_TILE);
          tma_load_2d(sX + sx * (MAXM * BK * 2), &tmap_x, &x_full[sx], kb * BK, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, p.Mpad, 0, 0);
      int it = 0, tile_i = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x, ++tile_i) {
        const int kb0 = (w / n_tiles) * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        if (!mbar_wait(acc_empty, (tile_i & 1) ^ 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % AB_STAGES;
          const uint32_t ph = (it / AB_STAGES) & 1;
          if (!mbar_wait(&a_full[s], ph, abort_flag, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          if (!mbar_wait(&x_full[s], ph, abort_flag, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A_TILE), x_base = smem_u32(sX + s * (MAXM * BK * 2));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16(tmem_base, make_smem_desc(a_base + k * 32, 16, 1024, 2), make_smem_desc(x_base + k * 32, 16, 1024, 2), idesc,
                      (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&a_empty[s]);
        }
        if (!ok) break;
        umma_commit(acc_full);
      }
    }
  } else {
    // ---------------- dequantise + epilogue ----------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;   // which 32-wide scale block of the 64-deep k-block
    const int r = q * 32 + lane;        // weight row inside the tile
    const int nsb = p.K / 32;           // scale blocks per weight row
    int it = 0, tile_i = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x, ++tile_i) {
      const int n0 = (w % n_tiles) * BN;
      const int kb0 = (w / n_tiles) * kb_per, kb1 = min(kb_total, kb0 + kb_per);
      const int row = n0 + r;
      const __nv_bfloat16* srow = p.scales + (size_t)min(row, p.N - 1) * nsb;
      __nv_bfloat16 sc_next = srow[kb0 * 2 + half];  // the scale is fetched one k-block ahead of its use
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const __nv_bfloat16 sc = sc_next;
        if (kb + 1 < kb1) sc_next = srow[(kb + 1) * 2 + half];
        const int si = it % IDX_STAGES, sa = it % AB_STAGES;
        if (!mbar_wait_warp(&idx_full[si], (it / IDX_STAGES) & 1, abort_flag, p.status, ERR_WAIT_FULL)) { ok = false; break; }
        if (!mbar_wait_warp(&a_empty[sa], ((it / AB_STAGES) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
        const __nv_bfloat162 sc2 = __halves2bfloat162(sc, sc);
        const uint8_t* src = sIdx + si * IDX_TILE + r * ROW_BYTES + half * (ROW_BYTES / 2);
        uint8_t* dst = sA + sa * A_TILE + (r >> 3) * 1024 + (r & 7) * 128;
        if (BITS == 2) {
          // 4-entry codebook (ternary {-1, 0, +1, 0} for SPARK / OIL1 weights, or the OIL2 levels): the four
          // scaled entries sit in one 64-bit register and every 2-bit code selects 16 bits of it
          const uint2 raw = *reinterpret_cast<const uint2*>(src);  // 32 weights
          const __nv_bfloat162 e01 = __hmul2(__floats2bfloat162_rn(p.codebook[0], p.codebook[1]), sc2);
          const __nv_bfloat162 e23 = __hmul2(__floats2bfloat162_rn(p.codebook[2], p.codebook[3]), sc2);
          const uint64_t tbl = (uint64_t)(*reinterpret_cast<const uint32_t*>(&e01)) | ((uint64_t)(*reinterpret_cast<const uint32_t*>(&e23)) << 32);
#pragma unroll
          for (int g = 0; g < 4; ++g) {  // 8 weights = 16 bits of codes
            const uint32_t codes = ((g < 2 ? raw.x : raw.y) >> (16 * (g & 1))) & 0xffffu;
            uint32_t o[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const uint32_t lo = (uint32_t)(tbl >> (16 * ((codes >> (4 * b)) & 3))) & 0xffffu;
              const uint32_t hi = (uint32_t)(tbl >> (16 * ((codes >> (4 * b + 2)) & 3))) << 16;
              o[b] = lo | hi;
            }
            *reinterpret_cast<uint4*>(dst + (((half * 4 + g) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else if (BITS == 4) {
          const uint4 raw = *reinterpret_cast<const uint4*>(src);  // 32 weights
          const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int g = 0; g < 4; ++g) {  // 8 weights = 4 bytes = one 16-byte chunk of bf16
            uint32_t o[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const uint32_t pair = lut[(((wds[g] >> (8 * b)) & 255) << 5) + lane];
              const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pair), sc2);
              o[b] = *reinterpret_cast<const uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(dst + (((half * 4 + g) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          const uint4 raw0 = *reinterpret_cast<const uint4*>(src), raw1 = *reinterpret_cast<const uint4*>(src + 16);
          const uint32_t wds[8] = {raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w};
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t o[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const uint32_t two = wds[g * 2 + (b >> 1)] >> (16 * (b & 1));
              const uint32_t lo = lut[((two & 255) << 5) + lane] & 0xffffu, hi = lut[(((two >> 8) & 255) << 5) + lane] << 16;
              const uint32_t pair = lo | hi;
              const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pair), sc2);
              o[b] = *reinterpret_cast<const uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(dst + (((half * 4 + g) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        mbar_arrive(&idx_empty[si]);
        fence_proxy_async_smem();
        mbar_arrive(&a_full[sa]);
      }
      if (!ok) break;
      // ---- epilogue: accumulator [weight row (lane), token (column)] -> out[token][n0 + row] ----
      if (!mbar_wait_warp(acc_full, tile_i & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16);
      const int chunks = p.Mpad / 16;
      for (int c = half; c < chunks; c += 2) {  // the two halves split the token columns
        uint32_t v[16];
        tmem_ld_32x16(t_row + c * 16, v);
        tmem_ld_wait();
        if (row < p.N) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = c * 16 + i;
            if (m < p.M) {
              float* dst = p.out + (size_t)m * p.ldo + row;
              if (p.multimem) asm volatile("multimem.red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(dst), "f"(__uint_as_float(v[i])) : "memory");
              else atomicAdd(dst, __uint_as_float(v[i]));
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty);
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
    tmem_dealloc(tmem_base, 256);
  }
}

// out_bf16[m, n] = bf16(acc[m, n] + bias[n] (+ residual[m, n])); clears acc for the next use.
__global__ void oil_gemm_finish_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
                                       __nv_bfloat16* __restrict__ out, long M, int N, int ld_acc, int ld_out, int ld_res, int clear) {
  const long m = blockIdx.y;
  for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < N; n += gridDim.x * blockDim.x) {
    float v = acc[m * ld_acc + n];
    if (clear) acc[m * ld_acc + n] = 0.f;
    if (bias) v += __bfloat162float(bias[n]);
    if (residual) v += __bfloat162float(residual[m * ld_res + n]);
    out[m * ld_out + n] = __float2bfloat16_rn(v);
  }
}

}  // namespace inv

using namespace inv;

// acc (fp32 [M, ldo]) must be zero on entry or hold a partial sum to add to. M <= 256, K % 64 == 0.
extern "C" int inv_oil_gemm(const void* x, int ldx, const void* idx, const void* scales, const float* codebook, int bits, float* acc, int ldo,
                            int M, int N, int K, int split_k, int* status, void* stream, int multimem) {
  using namespace og;
  if ((bits != 2 && bits != 4 && bits != 8) || M < 1 || M > MAXM || (K % 64) || (ldx % 8) || N < 1) return -ERR_BAD_ARG;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  OilGemmParams p;
  p.M = M; p.N = N; p.K = K; p.bits = bits;
  p.Mpad = (M + 15) / 16 * 16;
  p.scales = (const __nv_bfloat16*)scales;
  p.codebook = codebook;
  p.out = acc; p.ldo = ldo; p.status = status; p.multimem = multimem;
  const int n_tiles = (N + BN - 1) / BN, kb_total = K / BK;
  if (split_k <= 0) {  // several work units per SM (balance), each at least 4 k-blocks long
    split_k = (4 * num_sms + n_tiles - 1) / n_tiles;
    if (split_k > kb_total / 4) split_k = kb_total / 4 > 0 ? kb_total / 4 : 1;
  }
  if (split_k > kb_total) split_k = kb_total;
  {
    const int per = (kb_total + split_k - 1) / split_k;
    split_k = (kb_total + per - 1) / per;
  }
  p.split_k = split_k;
  CUtensorMap ti, tx;
  int rc;
  const int row_bytes = K * bits / 8;
  if ((rc = make_tmap_bytes(&ti, idx, (uint64_t)row_bytes, (uint64_t)N, BK * bits / 8, BN))) return rc;
  if ((rc = make_tmap_2d_bf16(&tx, x, (uint64_t)K, (uint64_t)M, (uint64_t)ldx, BK, (uint32_t)p.Mpad))) return rc;
  const int idx_tile = BN * BK * bits / 8;
  const int smem = AB_STAGES * (A_TILE + MAXM * BK * 2) + IDX_STAGES * idx_tile + 1024 + 256 * 32 * 4 + 512 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(oil_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(oil_gemm_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(oil_gemm_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    configured = true;
  }
  const int total = n_tiles * split_k;
  const int grid = total < num_sms ? total : num_sms;
  cudaStream_t st = (cudaStream_t)stream;
  if (bits == 2) oil_gemm_kernel<2><<<grid, THREADS, smem, st>>>(ti, tx, p);
  else if (bits == 4) oil_gemm_kernel<4><<<grid, THREADS, smem, st>>>(ti, tx, p);
  else oil_gemm_kernel<8><<<grid, THREADS, smem, st>>>(ti, tx, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_oil_gemm_finish(float* acc, const void* bias, const void* residual, void* out, long M, int N, int ld_acc, int ld_out,
                                   int ld_res, int clear, void* stream) {
  if (M <= 0) return 0;
  int gx = (N + 255) / 256;
  if (gx > 32) gx = 32;
  dim3 grid(gx, (unsigned)M);
  oil_gemm_finish_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(acc, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual,
                                                                  (__nv_bfloat16*)out, M, N, ld_acc, ld_out, ld_res, clear);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
