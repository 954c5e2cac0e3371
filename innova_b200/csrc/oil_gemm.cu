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
//   warp 0    TMA: raw index tiles (128 rows x 256 k, swizzled) and activation tiles (M x 64 k, 128B swizzle)
//   warp 1    MMA issuer: A operand from tensor memory, B (activations) from shared memory, two accumulators
//             [128 weight rows x M tokens] fp32 in TMEM
//   warps 2-9 dequantise, two groups of four warps on alternate index tiles: a thread owns a weight row, looks
//             the values up in a shared-memory table of bf16 pairs (OIL4: indexed by the byte, i.e. two weights
//             per lookup), multiplies by the block scale with packed bf16 math and stores the row's 64 values
//             per k-block into its lane of an A stage in tensor memory. The same warps run the epilogue.
// With `multimem` set the output pointer is an NVLS multicast address and the epilogue's reductions are
// multimem.red: the switch adds each partial sum into every rank's copy of the buffer, which turns a
// row-parallel (tensor-parallel) linear layer into GEMM + all-reduce in one kernel.
// Work is split stream-K: the (tile, k-block) pairs are cut into one equal contiguous range per SM, so every SM
// streams the same number of index bytes whatever N and K are, and the partial sums of a range are added to the
// fp32 output with reductions. Every wait is bounded.
#include "sm100_common.cuh"
#include "inv_api.h"

#include <mutex>

namespace inv {

int make_tmap_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                      uint32_t box_outer);

namespace og {
constexpr int BN = 128;     // weight rows per tile (MMA M)
constexpr int BK = 64;      // k-block: one A stage, one activation tile
constexpr int STG_PITCH = 132;  // floats per token row of the epilogue staging tile (128 weight rows + 4: conflict-free both ways)
constexpr int STG_TOK = 16;     // tokens per staging pass
constexpr int MAX_IDX_STAGES = 6;
constexpr int THREADS = 352;  // warp 0 TMA, warps 1 and 10 MMA issuers, warps 2-9 expand
constexpr int MAXM = 128;   // tokens per launch (MMA N); the host entry point splits larger M
constexpr int A_COL0 = 256;  // TMEM: accumulators in [0,256) (per buffer and issuer), A slots in [256,512)
}  // namespace og

struct OilGemmParams {
  int M, N, K, bits;  // bits = 2, 4 or 8
  int Mpad;           // M rounded up to 16
  const __nv_bfloat16* scales;
  const float* codebook;
  float* out;  // [M, N] fp32
  int ldo;
  int idx_stages;  // depth of the raw index ring: whatever shared memory is left, at most MAX_IDX_STAGES
  int dp_rounds;   // whole tiles per CTA before the stream-K tail (tile = round * gridDim.x + blockIdx.x)
  int* status;
  float* peers[8];  // mode 2: the same partial sums are added into each of these buffers (every rank's copy of the accumulator)
  int n_peers;
  int multimem;  // 1: out is an NVLS multicast address, every partial sum is added into all ranks' copies; 2: out may hold
                 // other ranks' partial sums (a peer's buffer): always add, never store; 3: reduce-scatter: column n is
                 // added into peers[n / owner_cols] only (the rank that owns that column range), so every partial sum
                 // crosses NVLink once instead of once per rank
  int owner_cols;
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
// Byte tensor map: `inner` bytes per row, `outer` rows; the box is one swizzle span wide (64 or 128 bytes).
static int make_tmap_bytes(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFnO enc = og_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = box_inner == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

// Expands one k-block of one weight row (64 weights) into 32 packed bf16 pairs, scaled. `raw` holds the row's
// index bytes for the k-block (16 B per 2-bit, 32 B per 4-bit, 64 B per 8-bit), `s0` / `s1` the two block scales.
template <int BITS>
__device__ __forceinline__ void expand_row(const uint4* raw, __nv_bfloat16 s0, __nv_bfloat16 s1, const uint32_t* lut, const float* cb, int lane,
                                           uint32_t* o) {
  if (BITS == 2) {
    // 4-entry codebook (ternary {-1, 0, +1, 0} for SPARK / OIL1 weights, or the OIL2 levels): the four scaled
    // entries sit in one 64-bit register and every 2-bit code selects 16 bits of it
    const uint32_t w[4] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __nv_bfloat162 sc2 = __halves2bfloat162(h ? s1 : s0, h ? s1 : s0);
      const __nv_bfloat162 e01 = __hmul2(__floats2bfloat162_rn(cb[0], cb[1]), sc2);
      const __nv_bfloat162 e23 = __hmul2(__floats2bfloat162_rn(cb[2], cb[3]), sc2);
      const uint64_t tbl = (uint64_t)(*reinterpret_cast<const uint32_t*>(&e01)) | ((uint64_t)(*reinterpret_cast<const uint32_t*>(&e23)) << 32);
#pragma unroll
      for (int j = 0; j < 2; ++j) {  // a 32-bit word = 16 codes = 8 output pairs
        const uint32_t codes = w[h * 2 + j];
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const uint32_t lo = (uint32_t)(tbl >> (16 * ((codes >> (4 * b)) & 3))) & 0xffffu;
          const uint32_t hi = (uint32_t)(tbl >> (16 * ((codes >> (4 * b + 2)) & 3))) << 16;
          o[h * 16 + j * 8 + b] = lo | hi;
        }
      }
    }
  } else if (BITS == 4) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __nv_bfloat162 sc2 = __halves2bfloat162(h ? s1 : s0, h ? s1 : s0);
      const uint32_t w[4] = {raw[h].x, raw[h].y, raw[h].z, raw[h].w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const uint32_t pair = lut[(((w[j] >> (8 * b)) & 255) << 5) + lane];
          const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pair), sc2);
          o[h * 16 + j * 4 + b] = *reinterpret_cast<const uint32_t*>(&v);
        }
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __nv_bfloat162 sc2 = __halves2bfloat162(h ? s1 : s0, h ? s1 : s0);
      const uint32_t w[8] = {raw[h * 2].x, raw[h * 2].y, raw[h * 2].z, raw[h * 2].w, raw[h * 2 + 1].x, raw[h * 2 + 1].y, raw[h * 2 + 1].z, raw[h * 2 + 1].w};
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const uint32_t two = w[j] >> (16 * b);
          const uint32_t lo = lut[((two & 255) << 5) + lane] & 0xffffu, hi = lut[(((two >> 8) & 255) << 5) + lane] << 16;
          const uint32_t pair = lo | hi;
          const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pair), sc2);
          o[h * 16 + j * 2 + b] = *reinterpret_cast<const uint32_t*>(&v);
        }
    }
  }
}

// Walks a CTA's work in order: `dp_rounds` whole tiles (tile = round * grid + cta, every batch of K), then its share of
// the stream-K tail: the (tile, batch) pairs of the remaining tiles, tile-major, cut into one equal contiguous range
// per CTA. One step = one batch (index tile). A segment is a maximal run of batches inside one tile.
struct OgCursor {
  int nb, grid, cta, dp_rounds, sk_tile0, sk_b1;
  int round, sk_b;
  int tile, bb, bb0, bb1;
  bool valid;
  __device__ __forceinline__ void next_segment() {
    if (round < dp_rounds) {
      tile = round * grid + cta;
      bb0 = 0; bb1 = nb;
      ++round;
      valid = true;
    } else if (sk_b < sk_b1) {
      const int t = sk_b / nb;
      bb0 = sk_b - t * nb;
      const int end = min(sk_b1, (t + 1) * nb);
      bb1 = bb0 + (end - sk_b);
      tile = sk_tile0 + t;
      sk_b = end;
      valid = true;
    } else {
      valid = false;
    }
    bb = bb0;
  }
  __device__ __forceinline__ OgCursor(int n_tiles, int nb_, int dp_rounds_) {
    nb = nb_; grid = gridDim.x; cta = blockIdx.x; dp_rounds = dp_rounds_;
    sk_tile0 = dp_rounds * grid;
    const long long total = (long long)(n_tiles - sk_tile0) * nb;
    sk_b = (int)(total * cta / grid);
    sk_b1 = (int)(total * (cta + 1) / grid);
    round = 0;
    next_segment();
  }
  __device__ __forceinline__ void advance() {
    if (++bb == bb1) next_segment();
  }
  __device__ __forceinline__ bool seg_first() const { return bb == bb0; }
  __device__ __forceinline__ bool seg_last() const { return bb + 1 == bb1; }
  __device__ __forceinline__ bool seg_full() const { return bb0 == 0 && bb1 == nb; }
};

// Build with -DOG_TRACE to record, for CTA 0 of the most recent launch, the SM clock at the phases of the kernel
// (inv_og_trace_read copies the stamps out): 0 entry, 1 set-up done, 2 first index TMA issued, 3 previous grid complete,
// 4 lookup table built, 5 first index tile landed, 6 first MMA inputs ready, 7 last MMA committed, 8 first epilogue
// starts, 9 last epilogue done, 10 exit.
#ifdef OG_TRACE
__device__ long long og_trace_buf[16];
#define OG_STAMP(i) do { if (blockIdx.x == 0) og_trace_buf[i] = clock64(); } while (0)
#define OG_STAMP_ONCE(i, flag) do { if (blockIdx.x == 0 && !(flag)) { og_trace_buf[i] = clock64(); flag = true; } } while (0)
#else
#define OG_STAMP(i) do {} while (0)
#define OG_STAMP_ONCE(i, flag) do {} while (0)
#endif

template <int BITS>
__global__ void __launch_bounds__(og::THREADS, 1)
oil_gemm_kernel(const __grid_constant__ CUtensorMap tmap_idx, const __grid_constant__ CUtensorMap tmap_x, const OilGemmParams p) {
  using namespace og;
  constexpr int KBB = BITS == 8 ? 2 : 4;           // k-blocks per index tile ("batch")
  constexpr int KB_BYTES = BK * BITS / 8;          // index bytes of one row in one k-block: 16, 32 or 64
  constexpr int KB_CHUNKS = KB_BYTES / 16;
  constexpr int ROWB = KBB * KB_BYTES;             // bytes per row of an index tile: 64 (2-bit) or 128
  constexpr int ROW_CHUNKS = ROWB / 16;
  constexpr int IDX_TILE = BN * ROWB;              // 8 or 16 KB
  const int X_TILE = p.Mpad * BK * 2;              // activation tile, also the stride of its ring
  const int IDX_STAGES = p.idx_stages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;                                  // 2 slots x KBB activation tiles (X_TILE is a multiple of 2 KB)
  uint8_t* sIdx = sX + 2 * KBB * X_TILE;               // IDX_STAGES x IDX_TILE (swizzled by TMA: 1 KB aligned)
  uint32_t* lut = reinterpret_cast<uint32_t*>(sIdx + IDX_STAGES * IDX_TILE);  // 256 entries x 32 bank copies
  float* stage = reinterpret_cast<float*>(lut + 256 * 32);  // epilogue staging: per group STG_TOK tokens x STG_PITCH
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage + 2 * STG_TOK * STG_PITCH);
  uint64_t* idx_full = bars;
  uint64_t* idx_empty = idx_full + MAX_IDX_STAGES;
  uint64_t* a_full = idx_empty + MAX_IDX_STAGES;  // [2]: slot g holds the batch expanded by group g (KBB k-blocks, 32 TMEM columns each)
  uint64_t* a_empty = a_full + 2;
  uint64_t* x_full = a_empty + 2;                 // [2]: the activation tiles of the same batch
  uint64_t* acc_full = x_full + 2;   // [buffer][owner group]: a barrier is always waited on by the same group, use after use
  uint64_t* acc_empty = acc_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* cb = reinterpret_cast<float*>(tmem_slot + 2);  // codebook copy, 256 entries

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int kb_total = p.K / BK;
  const int nb = (kb_total + KBB - 1) / KBB;  // batches per tile
  // Work split: whole tiles first (their result is stored), then a stream-K tail over the tiles that do not fill
  // another round of the grid (a CTA walks down K inside a tile and adds the finished segment into the fp32 output
  // with reductions). Every role below walks the same OgCursor.

  if (threadIdx.x == 0) OG_STAMP(0);
  if (threadIdx.x < (BITS == 8 ? 256 : (1 << BITS))) cb[threadIdx.x] = p.codebook[threadIdx.x];
  if (threadIdx.x == 0) {
    for (int s = 0; s < IDX_STAGES; ++s) {
      mbar_init(&idx_full[s], 1);
      mbar_init(&idx_empty[s], 4);  // the four warps of the group that expanded the tile
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&a_full[s], 4);
      mbar_init(&a_empty[s], 1);
      mbar_init(&x_full[s], 1);
      mbar_init(&acc_full[2 * s], 2);  // one commit per MMA issuer
      mbar_init(&acc_full[2 * s + 1], 2);
      mbar_init(&acc_empty[s], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_idx);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) OG_STAMP(1);
  [[maybe_unused]] bool og_once = false, og_once2 = false;

  if (warp == 0) {
    // lane 0 streams index tiles, lane 1 streams activation tiles; each runs ahead on its own ring
    if (lane == 0) {
      int si = 0;
      uint32_t ph = 1;
      for (OgCursor c(n_tiles, nb, p.dp_rounds); c.valid; c.advance()) {
        if (!mbar_wait(&idx_empty[si], ph, abort_flag, p.status, ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&idx_full[si], IDX_TILE);  // bytes past the end of K are filled with zeros and counted
        tma_load_2d(sIdx + si * IDX_TILE, &tmap_idx, &idx_full[si], c.bb * ROWB, c.tile * BN);
        OG_STAMP_ONCE(2, og_once);
        if (++si == IDX_STAGES) { si = 0; ph ^= 1; }
      }
    } else if (lane == 1) {
      // Programmatic dependent launch: this grid may start while the kernel that produces the activations is still
      // running. Everything that touches only the (static) weights runs ahead: index tiles are fetched and expanded
      // into tensor memory; the activation loads, and with them the MMAs and the epilogue, wait here for the
      // previous grid to complete.
      asm volatile("griddepcontrol.wait;" ::: "memory");
      OG_STAMP(3);
      int lb = 0;
      for (OgCursor c(n_tiles, nb, p.dp_rounds); c.valid; c.advance(), ++lb) {
        const int kb0 = c.bb * KBB, nkb = min(KBB, kb_total - kb0);
        const int slot = lb & 1;
        // the activation slot is released together with the A slot (same MMA commit)
        if (!mbar_wait(&a_empty[slot], ((lb >> 1) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&x_full[slot], nkb * X_TILE);
        for (int kk = 0; kk < nkb; ++kk) tma_load_2d(sX + (slot * KBB + kk) * X_TILE, &tmap_x, &x_full[slot], (kb0 + kk) * BK, 0);
      }
    }
  } else if (warp == 1 || warp == 10) {
    // Two MMA issuers, one per expanding group (a thread issues one tcgen05.mma per ~100 cycles whatever its size, so
    // with 64 tokens per instruction a single issuer would be the bottleneck). Issuer g multiplies the batches of
    // group g into its own accumulator; the epilogue adds the two. A thread runs at a few cycles per dependent
    // instruction, so the loop is kept lean: one pair of waits and one commit per batch, descriptors advanced by
    // additions.
    if (lane == 0) {
      const int g = warp == 1 ? 0 : 1;
      const uint32_t idesc = make_idesc_bf16(128, p.Mpad, 0, 0);
      const uint64_t xdesc0 = make_smem_desc(smem_u32(sX), 16, 1024, 2) + (uint64_t)(g * KBB) * (uint32_t)(X_TILE >> 4);
      const uint32_t x_step = (uint32_t)(X_TILE >> 4);
      const uint32_t a_col = tmem_base + A_COL0 + g * (KBB * 32);
      const int nbuf = p.Mpad <= 64 ? 2 : 1, accw = p.Mpad <= 64 ? 64 : 128;
      int lb = 0, seg = 0, seg_lb0 = 0;
      for (OgCursor c(n_tiles, nb, p.dp_rounds); c.valid; c.advance(), ++lb) {
        const int buf = nbuf == 2 ? (seg & 1) : 0, use = nbuf == 2 ? (seg >> 1) : seg;
        if (c.seg_first()) {
          seg_lb0 = lb;
          // both issuers wait here, owner of a batch in this segment or not: nobody may commit for this use of the
          // buffer before the previous use has been read out
          if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        }
        if ((lb & 1) == g) {
          const int nkb = min(KBB, kb_total - c.bb * KBB);
          const uint32_t ph = (lb >> 1) & 1;
          if (!mbar_wait(&a_full[g], ph, abort_flag, p.status, ERR_WAIT_FULL)) break;
          if (!mbar_wait(&x_full[g], ph, abort_flag, p.status, ERR_WAIT_FULL)) break;
          tc_fence_after();
          if (g == 0) OG_STAMP_ONCE(6, og_once);
          const uint32_t acc = tmem_base + (buf * 2 + g) * accw;
          umma_bf16_tmem_a(acc, a_col, xdesc0, idesc, (lb - seg_lb0) < 2 ? 0u : 1u);  // this issuer's first batch of the segment
#pragma unroll
          for (int k = 1; k < BK / 16; ++k) umma_bf16_tmem_a(acc, a_col + k * 8, xdesc0 + k * 2, idesc, 1u);
#pragma unroll
          for (int kk = 1; kk < KBB; ++kk) {
            if (kk < nkb) {
#pragma unroll
              for (int k = 0; k < BK / 16; ++k)  // 16 k = 8 packed columns of the A slot, 32 bytes of the swizzled activation row
                umma_bf16_tmem_a(acc, a_col + kk * 32 + k * 8, xdesc0 + (uint64_t)kk * x_step + k * 2, idesc, 1u);
            }
          }
          umma_commit(&a_empty[g]);
        }
        if (c.seg_last()) {
          umma_commit(&acc_full[buf * 2 + (lb & 1)]);  // the group that owns the last batch reads the segment out
          ++seg;
        }
      }
      if (g == 0) OG_STAMP(7);
    }
  } else if (warp >= 2 && warp < 10) {
    // lookup table: OIL4 -> bf16 pair (codebook[low nibble], codebook[high nibble]) per byte; OIL8 -> one bf16
    // entry e for lane l lives at lut[e * 32 + l]: every lane reads its own bank, whatever the indices are
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int r = q * 32 + lane;        // weight row inside the tile = TMEM lane
    const int nsb = p.K / 32;           // scale blocks per weight row
    const unsigned short* scales = reinterpret_cast<const unsigned short*>(p.scales);
    // block scales of a batch are fetched one own batch (two batches) ahead of their use
    unsigned short sc_next[2 * KBB];
    auto fetch_scales = [&](int t, int bbx) {
      const int kb0 = bbx * KBB;
      const unsigned short* row = scales + (size_t)min(t * BN + r, p.N - 1) * nsb + kb0 * 2;
#pragma unroll
      for (int j = 0; j < 2 * KBB; ++j) sc_next[j] = (kb0 * 2 + j < nsb) ? __ldg(row + j) : (unsigned short)0;
    };
    OgCursor pc(n_tiles, nb, p.dp_rounds);  // runs one own batch ahead of the main cursor
    if (grp == 1 && pc.valid) pc.advance();
    if (pc.valid) fetch_scales(pc.tile, pc.bb);  // in flight while the table is built
    if (BITS != 2) {
      // eight lanes write the 32 bank copies of one entry as 16-byte stores: a warp covers four entries (512 contiguous bytes)
      for (int e = (warp - 2) * 4 + (lane >> 3); e < 256; e += 32) {
        const uint32_t v = (BITS == 4) ? pack_bf16x2(cb[e & 15], cb[e >> 4]) : pack_bf16x2(cb[e], 0.f);
        *reinterpret_cast<uint4*>(lut + e * 32 + (lane & 7) * 4) = make_uint4(v, v, v, v);
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    if (threadIdx.x == 64) OG_STAMP(4);
    // ---------------- dequantise + epilogue ----------------
    // Two groups of four warps take alternate batches, so that one group's waits and barrier traffic overlap the
    // other group's table lookups. A thread owns weight row r of the tile: it reads the row's index bytes of the
    // whole batch, expands one k-block at a time into 32 registers of packed bf16 and stores them into its lane
    // of the A stage in tensor memory (the MMA reads A from there: no shared-memory round trip).
    const uint32_t t_lane = tmem_base + (uint32_t(q * 32) << 16);
    float* stg = stage + grp * (STG_TOK * STG_PITCH);
    [[maybe_unused]] const int gt = threadIdx.x - 64 - grp * 128;  // thread index inside the group
    const bool vec_ok = ((p.ldo & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    const int nbuf = p.Mpad <= 64 ? 2 : 1, accw = p.Mpad <= 64 ? 64 : 128;
    int seg = 0, lb = 0;
    uint32_t full_par = 0;  // bit b: parity of this group's next wait on acc_full[b * 2 + grp]
    bool ok = true;
    for (OgCursor c(n_tiles, nb, p.dp_rounds); ok && c.valid; c.advance(), ++lb) {
      const int nkb = min(KBB, kb_total - c.bb * KBB);
      const bool seg_end = c.seg_last();
      if ((lb & 1) == grp) {
        unsigned short sc[2 * KBB];
#pragma unroll
        for (int j = 0; j < 2 * KBB; ++j) sc[j] = sc_next[j];
        if (pc.valid) pc.advance();
        if (pc.valid) pc.advance();
        if (pc.valid) fetch_scales(pc.tile, pc.bb);
        const int si = lb % IDX_STAGES;
        if (!mbar_wait_warp(&idx_full[si], (lb / IDX_STAGES) & 1, abort_flag, p.status, ERR_WAIT_FULL)) { ok = false; break; }
        if (threadIdx.x == 64) OG_STAMP_ONCE(5, og_once);
        uint4 raw[ROW_CHUNKS];
        {
          const uint8_t* src = sIdx + si * IDX_TILE + r * ROWB;
          const int swz = (ROWB == 128) ? (r & 7) : ((r >> 1) & 3);  // the TMA swizzle of a 128- / 64-byte row
#pragma unroll
          for (int ch = 0; ch < ROW_CHUNKS; ++ch) raw[ch] = *reinterpret_cast<const uint4*>(src + ((ch ^ swz) << 4));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&idx_empty[si]);  // the tile lives in registers now
        // group g owns A slot g: free once the MMAs of this group's previous batch have completed
        if (!mbar_wait_warp(&a_empty[grp], ((lb >> 1) & 1) ^ 1, abort_flag, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < KBB; ++kk) {
          if (kk < nkb) {
            uint32_t o[32];
            const __nv_bfloat16_raw r0{sc[2 * kk]}, r1{sc[2 * kk + 1]};
            expand_row<BITS>(raw + kk * KB_CHUNKS, __nv_bfloat16(r0), __nv_bfloat16(r1), lut, cb, lane, o);
            tmem_st_32x32(t_lane + A_COL0 + (grp * KBB + kk) * 32, o);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[grp]);  // one arrival per warp
        if (seg_end) {
          // ---- segment end: accumulator [weight row (lane), token (column)] -> out[token][tile * 128 + row] ----
          // The tile is transposed through shared memory 32 tokens at a time, so that a thread ends up with four
          // consecutive weight rows of one token: one 16-byte store (whole tile) or vector reduction per thread.
          const bool full = c.seg_full() && p.multimem == 0;
          const int buf = nbuf == 2 ? (seg & 1) : 0, use = nbuf == 2 ? (seg >> 1) : seg;
          (void)use;
          if (!mbar_wait_warp(&acc_full[buf * 2 + grp], (full_par >> buf) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
          full_par ^= 1u << buf;
          tc_fence_after();
          if (gt == 0) OG_STAMP_ONCE(8, og_once2);
          const uint32_t t_acc = t_lane + (buf * 2 + grp) * accw, t_other = t_lane + (buf * 2 + (grp ^ 1)) * accw;
          const bool both = c.bb1 - c.bb0 >= 2;  // the other issuer contributed to this segment too
          for (int mh = 0; mh < p.Mpad; mh += STG_TOK) {
            uint32_t v[16], v2[16];
            tmem_ld_32x16(t_acc + mh, v);
            if (both) tmem_ld_32x16(t_other + mh, v2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) stg[j * STG_PITCH + r] = __uint_as_float(v[j]) + (both ? __uint_as_float(v2[j]) : 0.f);
            __syncwarp();  // a warp reads back only the 32 weight rows it wrote: no barrier across the group
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int e = k * 32 + lane, m = e >> 3, n4 = q * 32 + (e & 7) * 4;
              const int gm = mh + m, n = c.tile * BN + n4;
              if (gm < p.M && n < p.N) {
                const float4 val = *reinterpret_cast<const float4*>(stg + m * STG_PITCH + n4);
                float* o = p.out + (size_t)gm * p.ldo + n;
                if (vec_ok && n + 3 < p.N) {
                  if (p.multimem == 1)
                    asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(val.x), "f"(val.y), "f"(val.z), "f"(val.w) : "memory");
                  else if (p.multimem == 2) {
                    const size_t off = (size_t)gm * p.ldo + n;
                    for (int k = 0; k < p.n_peers; ++k)
                      asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p.peers[k] + off), "f"(val.x), "f"(val.y), "f"(val.z), "f"(val.w) : "memory");
                  } else if (p.multimem == 3) {  // owner_cols % 4 == 0: the four columns have one owner
                    asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p.peers[n / p.owner_cols] + (size_t)gm * p.ldo + n),
                                 "f"(val.x), "f"(val.y), "f"(val.z), "f"(val.w) : "memory");
                  }
                  else if (full)
                    *reinterpret_cast<float4*>(o) = val;
                  else
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(val.x), "f"(val.y), "f"(val.z), "f"(val.w) : "memory");
                } else {
                  const float vv[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
                  for (int z = 0; z < 4; ++z)
                    if (n + z < p.N) {
                      if (p.multimem == 1) asm volatile("multimem.red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(o + z), "f"(vv[z]) : "memory");
                      else if (p.multimem == 2) {
                        for (int k = 0; k < p.n_peers; ++k) atomicAdd(p.peers[k] + (size_t)gm * p.ldo + n + z, vv[z]);
                      } else if (p.multimem == 3) {
                        atomicAdd_system(p.peers[(n + z) / p.owner_cols] + (size_t)gm * p.ldo + n + z, vv[z]);
                      } else atomicAdd(o + z, vv[z]);
                    }
                }
              }
            }
            __syncwarp();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          if (gt == 0) OG_STAMP(9);
        }
      }
      if (seg_end) ++seg;
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) OG_STAMP(10);
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// out_bf16[m, n] = bf16(acc[m, n] + bias[n] (+ residual[m, n])); clears acc for the next use. Four columns per thread.
__global__ void oil_gemm_finish_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
                                       __nv_bfloat16* __restrict__ out, long M, int N, int ld_acc, int ld_out, int ld_res, int clear, int vec) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next GEMM may start fetching and expanding its weights
  const long m = blockIdx.y;
  if (vec) {
    for (int n = (blockIdx.x * blockDim.x + threadIdx.x) * 4; n < N; n += gridDim.x * blockDim.x * 4) {
      float4 v = *reinterpret_cast<float4*>(acc + m * ld_acc + n);
      if (clear) *reinterpret_cast<float4*>(acc + m * ld_acc + n) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (bias) {
        const uint2 b = *reinterpret_cast<const uint2*>(bias + n);
        v.x += __uint_as_float(b.x << 16); v.y += __uint_as_float(b.x & 0xffff0000u);
        v.z += __uint_as_float(b.y << 16); v.w += __uint_as_float(b.y & 0xffff0000u);
      }
      if (residual) {
        const uint2 b = *reinterpret_cast<const uint2*>(residual + m * ld_res + n);
        v.x += __uint_as_float(b.x << 16); v.y += __uint_as_float(b.x & 0xffff0000u);
        v.z += __uint_as_float(b.y << 16); v.w += __uint_as_float(b.y & 0xffff0000u);
      }
      *reinterpret_cast<uint2*>(out + m * ld_out + n) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    }
    return;
  }
  for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < N; n += gridDim.x * blockDim.x) {
    float v = acc[m * ld_acc + n];
    if (clear) acc[m * ld_acc + n] = 0.f;
    if (bias) v += __bfloat162float(bias[n]);
    if (residual) v += __bfloat162float(residual[m * ld_res + n]);
    out[m * ld_out + n] = __float2bfloat16_rn(v);
  }
}

// out[m, f] = bf16(silu(g) * u) with g = acc[m, f] (+ bias[f]), u = acc[m, F + f] (+ bias[F + f]); clears acc.
// The gate / up projection's finish and the SwiGLU in one pass. F % 4 == 0.
__global__ void oil_gemm_finish_swiglu_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int F,
                                              int ld_acc, int ld_out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const long m = blockIdx.y;
  for (int f = (blockIdx.x * blockDim.x + threadIdx.x) * 4; f < F; f += gridDim.x * blockDim.x * 4) {
    float4 g = *reinterpret_cast<float4*>(acc + m * ld_acc + f);
    float4 u = *reinterpret_cast<float4*>(acc + m * ld_acc + F + f);
    *reinterpret_cast<float4*>(acc + m * ld_acc + f) = make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(acc + m * ld_acc + F + f) = make_float4(0.f, 0.f, 0.f, 0.f);
    float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w}, r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (bias) {
        gv[i] += __bfloat162float(bias[f + i]);
        uv[i] += __bfloat162float(bias[F + f + i]);
      }
      // the unfused path rounds the projection to bf16 before the activation: same here
      const float gb = __bfloat162float(__float2bfloat16_rn(gv[i])), ub = __bfloat162float(__float2bfloat16_rn(uv[i]));
      r[i] = gb / (1.f + __expf(-gb)) * ub;
    }
    *reinterpret_cast<uint2*>(out + m * ld_out + f) = make_uint2(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]));
  }
}

// A barrier over peer flags at the head of a multi-CTA kernel, so that the barrier costs no launch of its own.
// `state` = {done, tickets} in this rank's memory: `done` is the epoch of the last completed use and is only written by
// the last CTA of a launch, so every CTA of the next launch reads the same value and derives the same epoch. CTA 0 raises
// this rank's word in every peer's flag set (everything this rank issued before the launch is complete: kernel boundary);
// every CTA waits, for at most a second, until all words of the local set have reached the epoch. `barrier_tail` is called
// by every CTA when it is done.
struct HeadBarrier {
  uint32_t* peer_flags[8];
  const uint32_t* local_flags;
  uint32_t* state;
  int* status;
};
__device__ __forceinline__ uint32_t barrier_head(const HeadBarrier& hb, int W, int rank) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    uint32_t d;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(d) : "l"(hb.state) : "memory");
    s_epoch = d + 1;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  if (blockIdx.x == 0 && threadIdx.x < W) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(hb.peer_flags[threadIdx.x] + rank), "r"(epoch) : "memory");
  }
  if (threadIdx.x < W) {
    uint64_t t0 = 0;
    uint32_t spins = 0, v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(hb.local_flags + threadIdx.x) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if ((++spins & 0xffu) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > 1000000000ull) {
          s_ok = 0;
          if (hb.status) atomicCAS(hb.status, 0, (int)ERR_WAIT_PEER);
          break;
        }
      }
    }
  }
  __syncthreads();
  return s_ok ? epoch : 0u;   // 0: a peer never arrived; the status word says so and the caller skips its work
}
__device__ __forceinline__ void barrier_tail(const HeadBarrier& hb, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(hb.state + 1, 1u) == gridDim.x - 1) {
      hb.state[1] = 0;
      // on a give-up the epoch still advances, so that the next use does not wait for this one's flags
      uint32_t d;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(d) : "l"(hb.state) : "memory");
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(hb.state), "r"(epoch ? epoch : d + 1) : "memory");
    }
  }
}
// x[m, :] = bf16(acc[m, :] + bias + residual[m, :]);  h[m, :] = bf16(rms_norm(x[m, :]) * w): the finish of a
// row-parallel projection with the next block's RMSNorm. One CTA of 256 threads per token; N % 4 == 0, N <= 16384.
__global__ void __launch_bounds__(256) oil_gemm_finish_norm_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ bias,
                                                                   const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ x_out,
                                                                   const __nv_bfloat16* __restrict__ w, float eps, __nv_bfloat16* __restrict__ h_out,
                                                                   int N, int ld_acc, int ld_x, int ld_res, int ld_h, int W, int rank,
                                                                   HeadBarrier hb) {
  constexpr int MAXV = 16;  // float4 groups per thread: 256 * 16 * 4 = 16384 columns
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const long m = blockIdx.x;
  uint32_t epoch = 1;
  if (hb.state != nullptr) {  // tensor parallel: every rank's GEMM has added its partial sums into this rank's accumulator
    epoch = barrier_head(hb, W, rank);
    if (epoch == 0) {
      barrier_tail(hb, 0);
      return;
    }
  }
  __shared__ float red[8];
  float4 xs[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int n = (i * 256 + threadIdx.x) * 4;
    if (n < N) {
      float4 v = *reinterpret_cast<float4*>(acc + m * ld_acc + n);
      *reinterpret_cast<float4*>(acc + m * ld_acc + n) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (bias) {
        const uint2 b = *reinterpret_cast<const uint2*>(bias + n);
        v.x += __uint_as_float(b.x << 16); v.y += __uint_as_float(b.x & 0xffff0000u);
        v.z += __uint_as_float(b.y << 16); v.w += __uint_as_float(b.y & 0xffff0000u);
      }
      if (residual) {
        const uint2 b = *reinterpret_cast<const uint2*>(residual + m * ld_res + n);
        v.x += __uint_as_float(b.x << 16); v.y += __uint_as_float(b.x & 0xffff0000u);
        v.z += __uint_as_float(b.y << 16); v.w += __uint_as_float(b.y & 0xffff0000u);
      }
      const uint32_t p0 = pack_bf16x2(v.x, v.y), p1 = pack_bf16x2(v.z, v.w);
      *reinterpret_cast<uint2*>(x_out + m * ld_x + n) = make_uint2(p0, p1);
      // the norm sees the rounded residual stream, as it does when it runs as a kernel of its own
      v.x = __uint_as_float(p0 << 16); v.y = __uint_as_float(p0 & 0xffff0000u);
      v.z = __uint_as_float(p1 << 16); v.w = __uint_as_float(p1 & 0xffff0000u);
      xs[i] = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / N + eps);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int n = (i * 256 + threadIdx.x) * 4;
    if (n < N) {
      const uint2 wb = *reinterpret_cast<const uint2*>(w + n);
      const float4 v = xs[i];
      const float r0 = v.x * rstd * __uint_as_float(wb.x << 16), r1 = v.y * rstd * __uint_as_float(wb.x & 0xffff0000u);
      const float r2 = v.z * rstd * __uint_as_float(wb.y << 16), r3 = v.w * rstd * __uint_as_float(wb.y & 0xffff0000u);
      *reinterpret_cast<uint2*>(h_out + m * ld_h + n) = make_uint2(pack_bf16x2(r0, r1), pack_bf16x2(r2, r3));
    }
  }
  if (hb.state != nullptr) barrier_tail(hb, epoch);
}

}  // namespace inv

using namespace inv;

// peer_flags / local_flags / state (all three, or none): the kernel starts with a barrier over that flag set (see HeadBarrier)
static HeadBarrier make_head_barrier(const uint64_t* peer_flags, void* local_flags, void* state, int W, int* status) {
  HeadBarrier hb;
  for (int r = 0; r < 8; ++r) hb.peer_flags[r] = peer_flags ? reinterpret_cast<uint32_t*>(peer_flags[r < W ? r : 0]) : nullptr;
  hb.local_flags = reinterpret_cast<const uint32_t*>(local_flags);
  hb.state = (peer_flags && local_flags) ? reinterpret_cast<uint32_t*>(state) : nullptr;
  hb.status = status;
  return hb;
}


static int oil_gemm_launch(const void* x, int ldx, const void* idx, const void* scales, const float* codebook, int bits, float* acc, int ldo,
                           int M, int N, int K, int* status, cudaStream_t st, int multimem, const uint64_t* peers = nullptr, int n_peers = 0,
                           size_t peer_off = 0, int owner_cols = 0) {
  using namespace og;
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
  p.n_peers = 0;
  p.owner_cols = owner_cols;
  for (int k = 0; k < 8; ++k) p.peers[k] = nullptr;
  if (multimem == 3) {
    p.n_peers = n_peers;
    for (int k = 0; k < n_peers; ++k) p.peers[k] = reinterpret_cast<float*>(peers[k]) + peer_off;
  }
  if (multimem == 2) {
    if (peers == nullptr) { p.peers[0] = acc; p.n_peers = 1; }
    else { p.n_peers = n_peers; for (int k = 0; k < n_peers; ++k) p.peers[k] = reinterpret_cast<float*>(peers[k]) + peer_off; }
  }
  const int kbb = bits == 8 ? 2 : 4;
  const int n_tiles = (N + BN - 1) / BN, kb_total = K / BK, nb = (kb_total + kbb - 1) / kbb;
  CUtensorMap ti, tx;
  int rc;
  const int row_bytes = K * bits / 8, rowb = kbb * BK * bits / 8;
  if ((rc = make_tmap_bytes(&ti, idx, (uint64_t)row_bytes, (uint64_t)N, rowb, BN))) return rc;
  if ((rc = make_tmap_2d_bf16(&tx, x, (uint64_t)K, (uint64_t)M, (uint64_t)ldx, BK, (uint32_t)p.Mpad))) return rc;
  const int idx_tile = BN * rowb;
  const int fixed = 1024 + 2 * kbb * p.Mpad * BK * 2 + 256 * 32 * 4 + 2 * STG_TOK * STG_PITCH * 4 + (2 * MAX_IDX_STAGES + 12) * 8 + 16 + 1024 + 64;
  int stages = (227 * 1024 - fixed) / idx_tile;
  if (stages > MAX_IDX_STAGES) stages = MAX_IDX_STAGES;
  stages &= ~1;  // even: a ring stage is then always read by the same expanding group, which sees every phase of its barrier
  if (stages < 2) return -ERR_BAD_ARG;
  p.idx_stages = stages;
  const int smem = fixed + stages * idx_tile;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(oil_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(oil_gemm_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(oil_gemm_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    configured = true;
  }
  // at least two batches per CTA (one per expanding group): shorter ranges cost more in prologue and reductions
  // than they win in parallelism
  const long long total = (long long)n_tiles * nb;
  int grid = (int)((total + 1) / 2);
  if (grid > num_sms) grid = num_sms;
  p.dp_rounds = n_tiles / grid;  // whole tiles while they fill rounds of the grid, the rest is the stream-K tail
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (bits == 2) e = cudaLaunchKernelEx(&cfg, oil_gemm_kernel<2>, ti, tx, p);
  else if (bits == 4) e = cudaLaunchKernelEx(&cfg, oil_gemm_kernel<4>, ti, tx, p);
  else e = cudaLaunchKernelEx(&cfg, oil_gemm_kernel<8>, ti, tx, p);
  return e == cudaSuccess ? 0 : -(int)e;
}

// acc (fp32 [M, ldo]) must be zero on entry or hold a partial sum to add to. M <= 256, K % 64 == 0.
extern "C" int inv_oil_gemm(const void* x, int ldx, const void* idx, const void* scales, const float* codebook, int bits, float* acc, int ldo,
                            int M, int N, int K, int split_k, int* status, void* stream, int multimem) {
  (void)split_k;  // the split is stream-K: equal (tile, batch) ranges per CTA
  if ((bits != 2 && bits != 4 && bits != 8) || M < 1 || M > 256 || (K % 64) || (ldx % 8) || N < 1) return -ERR_BAD_ARG;
  for (int m0 = 0; m0 < M; m0 += og::MAXM) {
    const int m = M - m0 < og::MAXM ? M - m0 : og::MAXM;
    const int rc = oil_gemm_launch((const __nv_bfloat16*)x + (size_t)m0 * ldx, ldx, idx, scales, codebook, bits, acc + (size_t)m0 * ldo, ldo, m, N, K,
                                   status, (cudaStream_t)stream, multimem);
    if (rc) return rc;
  }
  return 0;
}

// The same GEMM with the partial sums added into n_peers buffers (each rank's copy of a replicated accumulator, given
// as addresses that already include the column offset): one launch, the weights are read once.
extern "C" int inv_oil_gemm_peers(const void* x, int ldx, const void* idx, const void* scales, const float* codebook, int bits,
                                  const uint64_t* peers, int n_peers, int ldo, int M, int N, int K, int* status, void* stream) {
  if ((bits != 2 && bits != 4 && bits != 8) || M < 1 || M > 256 || (K % 64) || (ldx % 8) || N < 1 || n_peers < 1 || n_peers > 8) return -ERR_BAD_ARG;
  for (int m0 = 0; m0 < M; m0 += og::MAXM) {
    const int m = M - m0 < og::MAXM ? M - m0 : og::MAXM;
    const int rc = oil_gemm_launch((const __nv_bfloat16*)x + (size_t)m0 * ldx, ldx, idx, scales, codebook, bits,
                                   reinterpret_cast<float*>(peers[0]) + (size_t)m0 * ldo, ldo, m, N, K, status, (cudaStream_t)stream, 2, peers, n_peers,
                                   (size_t)m0 * ldo);
    if (rc) return rc;
  }
  return 0;
}

// Reduce-scatter form for tensor-parallel row-parallel layers: peers[r] is rank r's accumulator ([M, ldo] fp32, zero on
// entry); column n of every rank's partial product is added into peers[n / owner_cols] only. After a barrier rank r holds
// the complete sums of columns [r * owner_cols, (r + 1) * owner_cols).
extern "C" int inv_oil_gemm_rs(const void* x, int ldx, const void* idx, const void* scales, const float* codebook, int bits,
                               const uint64_t* peers, int W, int owner_cols, int ldo, int M, int N, int K, int* status, void* stream) {
  if ((bits != 2 && bits != 4 && bits != 8) || M < 1 || M > 256 || (K % 64) || (ldx % 8) || N < 1 || W < 1 || W > 8 || owner_cols < 4 ||
      (owner_cols % 4) || owner_cols * W < N)
    return -ERR_BAD_ARG;
  for (int m0 = 0; m0 < M; m0 += og::MAXM) {
    const int m = M - m0 < og::MAXM ? M - m0 : og::MAXM;
    const int rc = oil_gemm_launch((const __nv_bfloat16*)x + (size_t)m0 * ldx, ldx, idx, scales, codebook, bits,
                                   reinterpret_cast<float*>(peers[0]) + (size_t)m0 * ldo, ldo, m, N, K, status, (cudaStream_t)stream, 3, peers, W,
                                   (size_t)m0 * ldo, owner_cols);
    if (rc) return rc;
  }
  return 0;
}

namespace inv {
struct SlicePeers {
  __nv_bfloat16* x[8];   // every rank's copy of the [M, N] residual stream
  float* sumsq[8];       // every rank's [W, M] partial sums of squares
};
// Second half of the tensor-parallel all-reduce. This rank owns columns [c0, c0 + cols) of the reduced accumulator: add
// bias and residual there, round to bf16, write the slice into EVERY rank's copy of the residual stream together with the
// slice's sum of squares per row, clear the accumulator slice. One CTA per row.
__global__ void __launch_bounds__(256) tp_slice_finish_push_kernel(float* __restrict__ acc, int ld_acc, const __nv_bfloat16* __restrict__ bias,
                                                                   const __nv_bfloat16* __restrict__ residual, int ld_res, SlicePeers peers,
                                                                   int ld_x, int W, int rank, int c0, int cols, int M, HeadBarrier hb) {
  const int m = blockIdx.x;
  uint32_t epoch = 1;
  if (hb.state != nullptr) {  // every rank's GEMM has added its partial sums into this rank's accumulator slice
    epoch = barrier_head(hb, W, rank);
    if (epoch == 0) {
      barrier_tail(hb, 0);
      return;
    }
  }
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < cols; c += blockDim.x * 4) {
    const int n = c0 + c;
    float4 v = *reinterpret_cast<float4*>(acc + (size_t)m * ld_acc + n);
    *reinterpret_cast<float4*>(acc + (size_t)m * ld_acc + n) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) {
      const uint2 b = *reinterpret_cast<const uint2*>(bias + n);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
      const float2 f0 = __bfloat1622float2(b2[0]), f1 = __bfloat1622float2(b2[1]);
      v.x += f0.x; v.y += f0.y; v.z += f1.x; v.w += f1.y;
    }
    if (residual) {
      const uint2 r = *reinterpret_cast<const uint2*>(residual + (size_t)m * ld_res + n);
      const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&r);
      const float2 f0 = __bfloat1622float2(r2[0]), f1 = __bfloat1622float2(r2[1]);
      v.x += f0.x; v.y += f0.y; v.z += f1.x; v.w += f1.y;
    }
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    // the norm is taken of the rounded values, as the one-GPU finish pass does
    const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&o);
    const float2 g0 = __bfloat1622float2(q2[0]), g1 = __bfloat1622float2(q2[1]);
    ss += g0.x * g0.x + g0.y * g0.y + g1.x * g1.x + g1.y * g1.y;
    for (int k = 0; k < W; ++k) {
      const int r = (rank + k) % W;
      *reinterpret_cast<uint2*>(peers.x[r] + (size_t)m * ld_x + n) = o;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __shared__ float red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    for (int k = 0; k < W; ++k) peers.sumsq[(rank + k) % W][rank * M + m] = t;
  }
  if (hb.state != nullptr) barrier_tail(hb, epoch);
}
// h[m, :] = x[m, :] * rsqrt(sum_r sumsq[r][m] / N + eps) * w   (rows of the gathered residual stream)
__global__ void __launch_bounds__(256) tp_norm_apply_kernel(const __nv_bfloat16* __restrict__ x, int ld_x, const float* __restrict__ sumsq, int W,
                                                            int M, const __nv_bfloat16* __restrict__ w, float eps, __nv_bfloat16* __restrict__ h,
                                                            int ld_h, int N, int rank, HeadBarrier hb) {
  const int m = blockIdx.x;
  uint32_t epoch = 1;
  if (hb.state != nullptr) {  // every rank's slice and sums of squares have landed in this rank's copy
    epoch = barrier_head(hb, W, rank);
    if (epoch == 0) {
      barrier_tail(hb, 0);
      return;
    }
  }
  float t = 0.f;
  for (int r = 0; r < W; ++r) t += sumsq[r * M + m];
  const float rs = rsqrtf(t / (float)N + eps);
  for (int c = threadIdx.x * 4; c < N; c += blockDim.x * 4) {
    const uint2 xv = *reinterpret_cast<const uint2*>(x + (size_t)m * ld_x + c);
    const uint2 wv = *reinterpret_cast<const uint2*>(w + c);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
    const float2 a0 = __bfloat1622float2(x2[0]), a1 = __bfloat1622float2(x2[1]);
    const float2 g0 = __bfloat1622float2(w2[0]), g1 = __bfloat1622float2(w2[1]);
    uint2 o;
    o.x = pack_bf16x2(a0.x * rs * g0.x, a0.y * rs * g0.y);
    o.y = pack_bf16x2(a1.x * rs * g1.x, a1.y * rs * g1.y);
    *reinterpret_cast<uint2*>(h + (size_t)m * ld_h + c) = o;
  }
  if (hb.state != nullptr) barrier_tail(hb, epoch);
}
}  // namespace inv

extern "C" int inv_tp_slice_finish_push(float* acc, int ld_acc, const void* bias, const void* residual, int ld_res, const uint64_t* peer_x,
                                        const uint64_t* peer_sumsq, int ld_x, int W, int rank, int c0, int cols, int M,
                                        const uint64_t* peer_flags, void* local_flags, void* barrier_state, int* status, void* stream) {
  if (W < 1 || W > 8 || rank < 0 || rank >= W || (cols % 4) || (c0 % 4) || (ld_acc % 4) || (ld_res % 4) || (ld_x % 4) || M < 1) return -ERR_BAD_ARG;
  SlicePeers sp;
  for (int r = 0; r < 8; ++r) {
    sp.x[r] = reinterpret_cast<__nv_bfloat16*>(peer_x[r < W ? r : 0]);
    sp.sumsq[r] = reinterpret_cast<float*>(peer_sumsq[r < W ? r : 0]);
  }
  tp_slice_finish_push_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(acc, ld_acc, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual,
                                                                             ld_res, sp, ld_x, W, rank, c0, cols, M,
                                                                             make_head_barrier(peer_flags, local_flags, barrier_state, W, status));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_tp_norm_apply(const void* x, int ld_x, const float* sumsq, int W, int M, const void* w, float eps, void* h, int ld_h, int N,
                                 int rank, const uint64_t* peer_flags, void* local_flags, void* barrier_state, int* status, void* stream) {
  if ((N % 4) || (ld_x % 4) || (ld_h % 4) || M < 1 || W < 1 || W > 8) return -ERR_BAD_ARG;
  tp_norm_apply_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ld_x, sumsq, W, M, (const __nv_bfloat16*)w, eps,
                                                                      (__nv_bfloat16*)h, ld_h, N, rank,
                                                                      make_head_barrier(peer_flags, local_flags, barrier_state, W, status));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_oil_gemm_finish(float* acc, const void* bias, const void* residual, void* out, long M, int N, int ld_acc, int ld_out,
                                   int ld_res, int clear, void* stream) {
  if (M <= 0) return 0;
  const bool vec = (N % 4 == 0) && (ld_acc % 4 == 0) && (ld_out % 4 == 0) && (ld_res % 4 == 0) && ((uintptr_t)acc % 16 == 0) &&
                   ((uintptr_t)out % 8 == 0) && ((uintptr_t)bias % 8 == 0) && ((uintptr_t)residual % 8 == 0);
  const int per_block = vec ? 1024 : 256;
  int gx = (N + per_block - 1) / per_block;
  if (gx > 32) gx = 32;
  dim3 grid(gx, (unsigned)M);
  oil_gemm_finish_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(acc, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual,
                                                                  (__nv_bfloat16*)out, M, N, ld_acc, ld_out, ld_res, clear, vec ? 1 : 0);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// out[M, F] = silu(acc[:, :F] + bias[:F]) * (acc[:, F:] + bias[F:]); acc [M, 2F] is cleared.
extern "C" int inv_oil_gemm_finish_swiglu(float* acc, const void* bias, void* out, long M, int F, int ld_acc, int ld_out, void* stream) {
  if (M <= 0) return 0;
  if ((F % 4) || (ld_acc % 4) || (ld_out % 4) || ((uintptr_t)acc % 16) || ((uintptr_t)out % 8)) return -ERR_BAD_ARG;
  int gx = (F + 1023) / 1024;
  if (gx > 32) gx = 32;
  dim3 grid(gx, (unsigned)M);
  oil_gemm_finish_swiglu_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(acc, (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, F, ld_acc, ld_out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// x_out[M, N] = acc + bias + residual (bf16), h_out[M, N] = rms_norm(x_out) * norm_w; acc is cleared.
extern "C" int inv_oil_gemm_finish_norm(float* acc, const void* bias, const void* residual, void* x_out, const void* norm_w, float eps, void* h_out,
                                        long M, int N, int ld_acc, int ld_x, int ld_res, int ld_h, void* stream) {
  if (M <= 0) return 0;
  if ((N % 4) || N > 16384 || (ld_acc % 4) || (ld_x % 4) || (ld_res % 4) || (ld_h % 4) || ((uintptr_t)acc % 16) || ((uintptr_t)x_out % 8) ||
      ((uintptr_t)h_out % 8) || ((uintptr_t)bias % 8) || ((uintptr_t)residual % 8) || ((uintptr_t)norm_w % 8))
    return -ERR_BAD_ARG;
  oil_gemm_finish_norm_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(acc, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual,
                                                                              (__nv_bfloat16*)x_out, (const __nv_bfloat16*)norm_w, eps,
                                                                              (__nv_bfloat16*)h_out, N, ld_acc, ld_x, ld_res, ld_h, 1, 0,
                                                                              make_head_barrier(nullptr, nullptr, nullptr, 1, nullptr));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// The same as the closing pass of a tensor-parallel all-reduce: the kernel starts with a barrier over the ranks' flag set
// (every rank's GEMM epilogue has added its partial sums into this rank's accumulator), see HeadBarrier.
extern "C" int inv_oil_gemm_finish_norm_tp(float* acc, const void* bias, const void* residual, void* x_out, const void* norm_w, float eps,
                                           void* h_out, long M, int N, int ld_acc, int ld_x, int ld_res, int ld_h, int W, int rank,
                                           const uint64_t* peer_flags, void* local_flags, void* barrier_state, int* status, void* stream) {
  if (M <= 0) return 0;
  if ((N % 4) || N > 16384 || (ld_acc % 4) || (ld_x % 4) || (ld_res % 4) || (ld_h % 4) || ((uintptr_t)acc % 16) || ((uintptr_t)x_out % 8) ||
      ((uintptr_t)h_out % 8) || ((uintptr_t)bias % 8) || ((uintptr_t)residual % 8) || ((uintptr_t)norm_w % 8) || W < 1 || W > 8 ||
      peer_flags == nullptr || local_flags == nullptr || barrier_state == nullptr)
    return -ERR_BAD_ARG;
  oil_gemm_finish_norm_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(acc, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual,
                                                                              (__nv_bfloat16*)x_out, (const __nv_bfloat16*)norm_w, eps,
                                                                              (__nv_bfloat16*)h_out, N, ld_acc, ld_x, ld_res, ld_h, W, rank,
                                                                              make_head_barrier(peer_flags, local_flags, barrier_state, W, status));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

#ifdef OG_TRACE
extern "C" int inv_og_trace_read(long long* host16) {
  return (int)cudaMemcpyFromSymbol(host16, og_trace_buf, sizeof(long long) * 16);
}
#endif
