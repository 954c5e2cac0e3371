// Expert parallelism over peer memory: token dispatch and combine as direct NVLink stores / loads.
//
// Replaces the reference's ExpertParallel (every rank routes all tokens, runs its experts, all_reduce of the
// [T, D] output per layer; src/moe_model.cpp:484-641) and ExpertDispatcher::plan_all_to_all / dispatch_tokens /
// gather_results (src/expert_parallel.cpp:408-478) with a dropless all-to-all that moves each routed token once:
//
//   plan     one launch: every rank publishes its per-expert token counts into all peers' [W, E] table, the ranks meet
//            at a flag barrier, and each rank derives from its table alone (a) where in the owner's receive buffer its
//            tokens of expert e start (owner segments are 128-row aligned per expert, source ranks in rank order inside
//            a segment) and (b) its own receive layout (segment starts, real ends, expert of every 128-row tile)
//   dispatch one warp per (token, choice) stores the token's row straight into the owner GPU's receive buffer
//   combine  one warp per token loads its k expert outputs from the owners' output buffers, weights and sums
//
// Experts are assigned contiguously: expert e lives on rank e / experts_per_rank. Rows that would exceed the
// receive capacity get slot -1 and contribute nothing (capacity = W * T * K rows is dropless).
// The caller separates the phases with device-side barriers over peer flags.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {
namespace ep {

constexpr int MAX_E = 256, MAX_W = 8, ALIGN = 128;
struct Peers {
  void* p[MAX_W];
};

// table[W][E] -> send_base[E], local_offsets[epr + 1], real_end[epr] (one past the last real row of each local
// segment), tile_expert[max_tiles] (local expert id, -1 unused), cursor[E] = 0, recv_rows[0] = rows used on this rank.
__device__ void ep_plan_body(const int* __restrict__ table, int W, int rank, int E, int epr, int cap_rows, int* __restrict__ send_base,
                             int* __restrict__ local_offsets, int* __restrict__ real_end, int* __restrict__ tile_expert, int* __restrict__ cursor,
                             int max_tiles, int* __restrict__ recv_rows) {
  __shared__ int seg_start[MAX_E];   // start of expert e's segment inside its owner's buffer
  __shared__ int s_local[MAX_E + 1];
  if (threadIdx.x == 0) {
    for (int o = 0; o < W; ++o) {
      int run = 0;
      for (int le = 0; le < epr; ++le) {
        const int e = o * epr + le;
        seg_start[e] = run;
        int tot = 0;
        for (int s = 0; s < W; ++s) tot += table[s * E + e];
        if (o == rank) {
          s_local[le] = run;
          if (real_end != nullptr) real_end[le] = min(run + tot, cap_rows);
        }
        run += (tot + ALIGN - 1) / ALIGN * ALIGN;
      }
      if (o == rank) s_local[epr] = run;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < rank; ++s) before += table[s * E + e];
    send_base[e] = seg_start[e] + before;
    cursor[e] = 0;
  }
  for (int le = threadIdx.x; le <= epr; le += blockDim.x) local_offsets[le] = min(s_local[le], cap_rows);
  if (threadIdx.x == 0) recv_rows[0] = min(s_local[epr], cap_rows);
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * ALIGN;
    int ex = -1;
    for (int le = 0; le < epr; ++le)
      if (row >= s_local[le] && row < s_local[le + 1]) ex = le;
    tile_expert[t] = ex;
  }
}

// Counts exchange, the barrier behind it and the plan in ONE launch: publish this rank's counts into every peer's table,
// raise this rank's word of every peer's flag set to the next epoch (the epoch counter lives on the device), wait (at most
// a second; the status word records a give-up) until every peer's word has reached it, then plan from the local table.
__global__ void __launch_bounds__(256) ep_exchange_plan_kernel(Peers tables, Peers flags, uint32_t* __restrict__ local_flags,
                                                               uint32_t* __restrict__ counter, const int* __restrict__ counts, int W, int rank,
                                                               int E, int epr, int cap_rows, int* __restrict__ send_base,
                                                               int* __restrict__ local_offsets, int* __restrict__ real_end,
                                                               int* __restrict__ tile_expert, int* __restrict__ cursor, int max_tiles,
                                                               int* __restrict__ recv_rows, int* __restrict__ status) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  for (int i = threadIdx.x; i < E * W; i += blockDim.x) {
    const int r = i / E, e = i % E;
    reinterpret_cast<int*>(tables.p[r])[rank * E + e] = counts[e];
  }
  if (threadIdx.x == 0) {
    s_epoch = atomicAdd(counter, 1u) + 1u;
    s_ok = 1;
  }
  __threadfence_system();
  __syncthreads();
  const uint32_t epoch = s_epoch;
  if (threadIdx.x < W) {
    uint32_t* f = reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    uint64_t t0 = 0;
    uint32_t spins = 0, v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local_flags + threadIdx.x) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if ((++spins & 0xffu) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > 1000000000ull) {
          s_ok = 0;
          if (status) atomicCAS(status, 0, (int)inv::ERR_WAIT_PEER);
          break;
        }
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;   // a peer never arrived: leave the plan untouched, the host reads the status word
  ep_plan_body(reinterpret_cast<const int*>(tables.p[rank]), W, rank, E, epr, cap_rows, send_base, local_offsets, real_end, tile_expert, cursor,
               max_tiles, recv_rows);
}

// assign = 1: claim a row (send_base[e] + cursor[e]++) and remember it in slot; assign = 0: reuse slot.
// scale_w != nullptr multiplies the row by the routing weight (combine backward).
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                                                          const int* __restrict__ send_base, int* __restrict__ cursor, int* __restrict__ slot,
                                                          const float* __restrict__ scale_w, Peers recv, int T, int K, int D, int epr, int cap_rows,
                                                          int assign) {
  const int lane = threadIdx.x & 31;
  const long id = blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long)T * K) return;
  const int t = (int)(id / K);
  const int e = topk_idx[id];
  int s;
  if (assign) {
    if (lane == 0) {
      s = send_base[e] + atomicAdd(&cursor[e], 1);
      if (s >= cap_rows) s = -1;
      slot[id] = s;
    }
    s = __shfl_sync(0xffffffffu, s, 0);
  } else {
    s = slot[id];
  }
  if (s < 0) return;
  const float w = scale_w ? scale_w[id] : 1.f;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * D);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recv.p[e / epr]) + (size_t)s * D);
  for (int i = lane; i < D / 8; i += 32) {
    uint4 v = src[i];
    if (scale_w) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(f.x * w, f.y * w);
      }
    }
    dst[i] = v;
  }
}

// out[t] = sum_k w[t,k] * y_owner[slot[t,k]] (+ residual[t]); weights == nullptr: plain sum.
// y_copy != nullptr keeps the k pulled rows ([T*K, D]) for the backward pass.
__global__ void __launch_bounds__(256) ep_combine_kernel(Peers ybuf, const int* __restrict__ topk_idx, const int* __restrict__ slot,
                                                         const float* __restrict__ weights, const __nv_bfloat16* __restrict__ residual,
                                                         __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ y_copy, int T, int K, int D,
                                                         int epr) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  for (int i = lane; i < D / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (residual) {
      const uint4 r = reinterpret_cast<const uint4*>(residual + (size_t)t * D)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int k = 0; k < K; ++k) {
      const size_t id = (size_t)t * K + k;
      const int s = slot[id];
      uint4 v = make_uint4(0, 0, 0, 0);
      if (s >= 0) v = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(ybuf.p[topk_idx[id] / epr]) + (size_t)s * D)[i];
      if (y_copy) reinterpret_cast<uint4*>(y_copy + id * D)[i] = v;
      const float w = weights ? weights[id] : 1.f;
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += w * f.x;
        acc[2 * j + 1] += w * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (size_t)t * D)[i] = o;
  }
}

// Zero the padding rows of this rank's receive segments (rows between an expert's last real row and the next 128-row
// boundary): the only rows of the receive buffer that the expert GEMMs read and that no peer writes.
__global__ void __launch_bounds__(256) ep_zero_pad_kernel(__nv_bfloat16* __restrict__ stage, const int* __restrict__ local_offsets,
                                                          const int* __restrict__ real_end, int D) {
  const int le = blockIdx.y;
  const int lo = real_end[le], hi = local_offsets[le + 1];
  const long vec = D / 8;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < (long)(hi - lo) * vec; i += (long)gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(stage + (size_t)lo * D)[i] = make_uint4(0, 0, 0, 0);
}

// dst[r] = src[r] for r < min(max_rows, *rows_dev); rows of row_bytes (a multiple of 16).
__global__ void __launch_bounds__(256) copy_rows_dev_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long vec_per_row, long max_rows,
                                                            const int* __restrict__ rows_dev) {
  const long total = min(max_rows, (long)*rows_dev) * vec_per_row;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) dst[i] = src[i];
}

static int fill(Peers& pp, const uint64_t* host_ptrs, int W) {
  if (W < 1 || W > MAX_W) return -1;
  for (int i = 0; i < MAX_W; ++i) pp.p[i] = i < W ? reinterpret_cast<void*>(host_ptrs[i]) : nullptr;
  return 0;
}

}  // namespace ep
}  // namespace inv

using namespace inv::ep;
#define EP_RET()                            \
  do {                                      \
    cudaError_t e = cudaGetLastError();     \
    return e == cudaSuccess ? 0 : -(int)e;  \
  } while (0)

extern "C" int inv_ep_dispatch(const void* x, const int* topk_idx, const int* send_base, int* cursor, int* slot, const float* scale_w,
                               const uint64_t* peer_recv, int W, int T, int K, int D, int experts_per_rank, int cap_rows, int assign, void* stream) {
  Peers r;
  if (fill(r, peer_recv, W) || D % 8) return -inv::ERR_BAD_ARG;
  if (T <= 0) return 0;
  const long warps = (long)T * K;
  ep_dispatch_kernel<<<(int)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, topk_idx, send_base, cursor, slot, scale_w, r,
                                                                              T, K, D, experts_per_rank, cap_rows, assign);
  EP_RET();
}
extern "C" int inv_ep_combine(const uint64_t* peer_y, int W, const int* topk_idx, const int* slot, const float* weights, const void* residual,
                              void* out, void* y_copy, int T, int K, int D, int experts_per_rank, void* stream) {
  Peers y;
  if (fill(y, peer_y, W) || D % 8) return -inv::ERR_BAD_ARG;
  if (T <= 0) return 0;
  ep_combine_kernel<<<(T + 7) / 8, 256, 0, (cudaStream_t)stream>>>(y, topk_idx, slot, weights, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out,
                                                                  (__nv_bfloat16*)y_copy, T, K, D, experts_per_rank);
  EP_RET();
}
extern "C" int inv_ep_zero_pad(void* stage, const int* local_offsets, const int* real_end, int experts_per_rank, int D, void* stream) {
  if (experts_per_rank < 1 || experts_per_rank > MAX_E || D % 8) return -inv::ERR_BAD_ARG;
  ep_zero_pad_kernel<<<dim3(8, experts_per_rank), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)stage, local_offsets, real_end, D);
  EP_RET();
}
extern "C" int inv_ep_exchange_plan(const uint64_t* peer_tables, const uint64_t* peer_flags, void* local_flags, void* counter, const int* counts,
                                    int W, int rank, int E, int experts_per_rank, int cap_rows, int* send_base, int* local_offsets, int* real_end,
                                    int* tile_expert, int* cursor, int max_tiles, int* recv_rows, int* status, void* stream) {
  Peers t, f;
  if (fill(t, peer_tables, W) || fill(f, peer_flags, W) || E < 1 || E > MAX_E || experts_per_rank * W != E) return -inv::ERR_BAD_ARG;
  ep_exchange_plan_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(t, f, (uint32_t*)local_flags, (uint32_t*)counter, counts, W, rank, E,
                                                               experts_per_rank, cap_rows, send_base, local_offsets, real_end, tile_expert, cursor,
                                                               max_tiles, recv_rows, status);
  EP_RET();
}
extern "C" int inv_copy_rows_dev(void* dst, const void* src, long row_bytes, long max_rows, const int* rows_dev, void* stream) {
  if (row_bytes % 16 || rows_dev == nullptr) return -inv::ERR_BAD_ARG;
  if (max_rows <= 0) return 0;
  copy_rows_dev_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>((uint4*)dst, (const uint4*)src, row_bytes / 16, max_rows, rows_dev);
  EP_RET();
}
