// Shared pieces of the tcgen05 GEMM kernels: launch parameters and the register-level epilogue.
#pragma once
#include "sm100_common.cuh"
#include "inv_api.h"
#include "side_job.cuh"

namespace inv {

struct GemmParams {
  int M, N, K;
  int split_k;
  void* C;
  int ldc;
  int c_f32;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;
  int ld_aux;
  __nv_bfloat16* aux_out;
  int epilogue;
  float alpha;
  int* status;
  // Grouped (mixture-of-experts) operation, single-CTA kernel only. Rows of A are grouped in
  // segments that start on multiples of 128 rows (csrc/moe.cu).
  //   1: C[rows of group e] = A[rows of group e] * B_e^T. tile_expert[m_tile] gives e (-1: unused tile);
  //      B_e starts group_rows_b rows further into the stacked B per group; bias likewise (group_stride_bias).
  //   2: C_e[M, N] += A[rows of e]^T-style reduction over the rows of group e only (expert weight
  //      gradients): the k range of group e comes from group_offsets[e..e+1]; C_e = C + e * group_stride_c.
  int group_mode;
  int num_groups;
  const int* tile_expert;
  const int* group_offsets;
  int group_rows_b;
  int group_stride_bias;
  long group_stride_c;
  // Collectives fused into the single-CTA kernel (tensor / sequence parallel layers, sharded weights).
  // All-gather -> GEMM: the gathered operand (ag_operand 0: A rows, 1: B rows) consists of ag_world shards of
  // ag_shard_rows rows. This rank's shard is already in place in the local full-size buffer the tensor map
  // covers (ag_dst); the first ag_copy_ctas CTAs of the grid pull the other shards out of the peers' buffers
  // (ag_src[r], same layout) tile by tile and publish ag_flags[tile] = ag_epoch; the GEMM CTAs visit tiles
  // local shard first, then in the order the copies arrive, and wait (bounded) on a tile's flag before its
  // first TMA load. Each remote tile crosses NVLink once and is then read from local memory / L2.
  int ag_world = 0, ag_rank = 0, ag_operand = 0, ag_shard_rows = 0, ag_copy_ctas = 0, ag_ld = 0;
  const void* ag_src[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  void* ag_dst = nullptr;
  uint32_t* ag_flags = nullptr;
  uint32_t ag_epoch = 0;
  // GEMM -> reduce-scatter: C's rows are rs_world shards of rs_shard_rows rows and shard r is owned by rank r.
  // The fp32 epilogue adds (red.global.add) each tile into the owner's buffer rs_dst[r] ([rs_shard_rows, ldc]),
  // over NVLink for remote owners; every rank's partial products meet there. Owners are visited starting
  // after this rank so the ranks never all write to the same destination.
  int rs_world = 0, rs_rank = 0, rs_shard_rows = 0;
  float* rs_dst[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  // A collective of the sharded data-parallel engine carried by the first side.n_ctas CTAs of the grid (side_job.cuh);
  // CTA-pair kernel only, not together with a fused all-gather.
  SideJob side = {};
};

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows of `ld` elements; 128B swizzle.
int make_tmap_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                      uint32_t box_outer);

// One thread's 32 consecutive accumulator columns (row `row`, columns col0..col0+31) through the
// fused epilogue and out to memory. `r` holds the raw fp32 bits read from TMEM.
// bf16 results go either straight to global memory (stg_c == nullptr) or into this thread's 128-byte
// row of a 32-row x 64-column staging box in shared memory (128B swizzle), from which the warp
// issues one TMA store; `sub` says which 32-column half of the box these columns are.
// `stg_in` (optional): this thread's 128-byte row of a box of the same shape and swizzle that a TMA load filled with
// the epilogue's second operand (residual / pre-activation); it may be the same box as `stg_c` (each thread reads its
// own 16-byte slots before it overwrites them).
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmParams& p, int row, bool row_ok, int col0, const uint32_t* r,
                                                    uint8_t* stg_c = nullptr, uint8_t* stg_aux = nullptr, int sub = 0, int lane = 0,
                                                    const uint8_t* stg_in = nullptr) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
    if (p.bias != nullptr) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (col0 + g * 8 < p.N) {
          uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + g * 8));
          const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(b2[j]);
            v[g * 8 + 2 * j] += f.x;
            v[g * 8 + 2 * j + 1] += f.y;
          }
        }
      }
    }
    if (row_ok) {
      if (p.epilogue == EPI_GELU_DG) {
        // both the activation and its derivative from one tanh per pair; the derivative is what the backward pass needs
        float dgv[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 d = gelu_tanh_grad_pair(v[i], v[i + 1]);
          const float2 y = gelu_tanh_pair(v[i], v[i + 1]);   // the common subexpressions (clamp, cubic, tanh) are merged by the compiler
          dgv[i] = d.x; dgv[i + 1] = d.y;
          v[i] = y.x; v[i + 1] = y.y;
        }
        __nv_bfloat16* ap = p.aux_out + (size_t)row * p.ld_aux + col0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (col0 + g * 8 < p.N) {
            uint4 o;
            o.x = pack_bf16x2(dgv[g * 8 + 0], dgv[g * 8 + 1]);
            o.y = pack_bf16x2(dgv[g * 8 + 2], dgv[g * 8 + 3]);
            o.z = pack_bf16x2(dgv[g * 8 + 4], dgv[g * 8 + 5]);
            o.w = pack_bf16x2(dgv[g * 8 + 6], dgv[g * 8 + 7]);
            if (stg_aux) *reinterpret_cast<uint4*>(stg_aux + (((sub * 4 + g) ^ (lane & 7)) << 4)) = o;
            else *reinterpret_cast<uint4*>(ap + g * 8) = o;
          }
        }
      } else if (p.epilogue == EPI_GELU) {
        if (p.aux_out != nullptr) {
          __nv_bfloat16* ap = p.aux_out + (size_t)row * p.ld_aux + col0;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (col0 + g * 8 < p.N) {
              uint4 o;
              o.x = pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]);
              o.y = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
              o.z = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]);
              o.w = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
              if (stg_aux) *reinterpret_cast<uint4*>(stg_aux + (((sub * 4 + g) ^ (lane & 7)) << 4)) = o;
              else *reinterpret_cast<uint4*>(ap + g * 8) = o;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 y = gelu_tanh_pair(v[i], v[i + 1]);
          v[i] = y.x;
          v[i + 1] = y.y;
        }
      } else if (INV_EPI_READS_AUX(p.epilogue)) {
        const __nv_bfloat16* ap = p.aux_in + (size_t)row * p.ld_aux + col0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (col0 + g * 8 < p.N) {
            const uint4 av = stg_in ? *reinterpret_cast<const uint4*>(stg_in + (((sub * 4 + g) ^ (lane & 7)) << 4))
                                    : *reinterpret_cast<const uint4*>(ap + g * 8);
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 f = __bfloat1622float2(a2[j]);
              if (p.epilogue == EPI_DGELU) {
                const float2 d = gelu_tanh_grad_pair(f.x, f.y);
                v[g * 8 + 2 * j] *= d.x;
                v[g * 8 + 2 * j + 1] *= d.y;
              } else if (p.epilogue == EPI_MUL) {
                v[g * 8 + 2 * j] *= f.x;
                v[g * 8 + 2 * j + 1] *= f.y;
              } else {
                v[g * 8 + 2 * j] += f.x;
                v[g * 8 + 2 * j + 1] += f.y;
              }
            }
          }
        }
      }
      if (p.c_f32) {
        float* cp = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
        if (p.epilogue == EPI_ATOMIC) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (col0 + g * 4 < p.N) {
              if (p.rs_world > 1)  // the destination may be another GPU's memory: system scope
                asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + g * 4), "f"(v[g * 4]),
                             "f"(v[g * 4 + 1]), "f"(v[g * 4 + 2]), "f"(v[g * 4 + 3])
                             : "memory");
              else
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + g * 4), "f"(v[g * 4]),
                             "f"(v[g * 4 + 1]), "f"(v[g * 4 + 2]), "f"(v[g * 4 + 3])
                             : "memory");
            }
          }
        } else {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (col0 + g * 4 < p.N)
              *reinterpret_cast<float4*>(cp + g * 4) = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
          }
        }
      } else {
        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (col0 + g * 8 < p.N) {
            uint4 o;
            o.x = pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]);
            o.y = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
            o.z = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]);
            o.w = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
            if (stg_c) *reinterpret_cast<uint4*>(stg_c + (((sub * 4 + g) ^ (lane & 7)) << 4)) = o;
            else *reinterpret_cast<uint4*>(cp + g * 8) = o;
          }
        }
      }
    }
}

// TMA store of a shared-memory box (128B swizzle) into a 2-D bf16 tensor; rows / columns outside
// the tensor are clipped by the hardware.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the shared memory of every committed store group of this thread has been read.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ----- fused all-gather: flags, bounded tile wait, copier CTAs (shared by the one- and two-CTA kernels) -----
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for a gathered tile; afterwards the async proxy (TMA) may read what the copier's ordinary stores wrote.
__device__ __forceinline__ bool ag_wait_tile(const GemmParams& p, int tile, volatile int* abort_flag) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (ld_acquire_gpu_u32(p.ag_flags + tile) != p.ag_epoch) {
    if ((++spins & 0xffu) == 0) {  // the global timer is slow to read: look at it only now and then
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > INV_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (p.status) atomicExch(p.status, ERR_WAIT_PEER);
        return false;
      }
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}
// Copier CTAs: remote shards, nearest peer first, one tile (`tile_rows` rows of K elements) per step. One thread drives the
// copy engine: bulk asynchronous copies peer memory -> shared memory -> local memory through a ring of 32 KB slots, four
// loads in flight ahead of the stores (about 160 KB per CTA: NVLink round trips are microseconds long, so a CTA moving
// registers' worth of data at a time would reach a few GB/s only). No cluster multicast.
static __device__ __noinline__ void ag_copier(const GemmParams& p, int tile_rows, uint8_t* ring, uint64_t* bars, volatile int* abort_flag) {
  constexpr int SLOTS = 6, AHEAD = 4, CH = 32768;
  if (threadIdx.x != 0) return;
  for (int s = 0; s < SLOTS; ++s) mbar_init(&bars[s], 1);
  *abort_flag = 0;
  fence_barrier_init();
  const int per = p.ag_shard_rows / tile_rows;
  const int remote_tiles = (p.ag_world - 1) * per;
  const size_t row_bytes = (size_t)p.K * 2, ld_bytes = (size_t)p.ag_ld * 2;
  const bool flat = row_bytes == ld_bytes;  // the tile is one contiguous range: copy it in 32 KB pieces, else row by row
  const size_t tile_bytes = (size_t)tile_rows * row_bytes;
  const int pieces_per_row = (int)((row_bytes + CH - 1) / CH);
  const int nch = flat ? (int)((tile_bytes + CH - 1) / CH) : tile_rows * pieces_per_row;
  uint32_t gi = 0;  // loads issued so far: slot = gi % SLOTS, use = gi / SLOTS
  uint32_t gw = 0;  // loads waited for so far
  for (int c = blockIdx.x; c < remote_tiles; c += p.ag_copy_ctas) {
    const int r = (p.ag_rank + 1 + c / per) % p.ag_world;
    const int tile = r * per + c % per;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ag_src[r]) + (size_t)tile * tile_rows * ld_bytes;
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.ag_dst) + (size_t)tile * tile_rows * ld_bytes;
    auto piece = [&](int i, size_t& off, uint32_t& bytes) {
      if (flat) {
        off = (size_t)i * CH;
        bytes = (uint32_t)(tile_bytes - off < (size_t)CH ? tile_bytes - off : (size_t)CH);
      } else {
        const int row = i / pieces_per_row, pc = i % pieces_per_row;
        const size_t col = (size_t)pc * CH;
        off = (size_t)row * ld_bytes + col;
        bytes = (uint32_t)(row_bytes - col < (size_t)CH ? row_bytes - col : (size_t)CH);
      }
    };
    bool ok = true;
    for (int i = 0; ok && i < nch + AHEAD; ++i) {
      if (i < nch) {
        // the slot's previous store must have read its data: at most SLOTS - AHEAD - 1 newer stores may still be pending
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        size_t off;
        uint32_t bytes;
        piece(i, off, bytes);
        const uint32_t slot = gi % SLOTS;
        mbar_expect_tx(&bars[slot], bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(ring + slot * CH)),
                     "l"(src + off), "r"(bytes), "r"(smem_u32(&bars[slot]))
                     : "memory");
        ++gi;
      }
      if (i >= AHEAD) {
        size_t off;
        uint32_t bytes;
        piece(i - AHEAD, off, bytes);
        const uint32_t slot = gw % SLOTS;
        if (!mbar_wait(&bars[slot], (gw / SLOTS) & 1, abort_flag, p.status, ERR_WAIT_PEER)) { ok = false; break; }
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + off), "r"(smem_u32(ring + slot * CH)), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        ++gw;
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // also on the way out after a failed wait: no store of ours stays in flight
    if (!ok) {  // give the loads still in flight a bounded time to land before the shared memory goes away
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      return;
    }
    __threadfence();
    asm volatile("fence.proxy.async;" ::: "memory");
    st_release_gpu_u32(p.ag_flags + tile, p.ag_epoch);
  }
}


}  // namespace inv
