// Collectives written as kernels over peer memory (NVLink 5 / NVSwitch), fused with the compute
// that follows them.
//
//   fsdp_reduce_kernel       reduce-scatter of the fp32 gradient: every rank pulls its shard from all
//                            peers with plain P2P loads, sums in a fixed rank order, keeps the sum
//                            local, and publishes its partial sum of squares to every peer.
//   fsdp_adamw_push_kernel   global-norm clip + AdamW on the owned shard + bf16 write of the new
//                            parameters straight into every peer's parameter buffer (the all-gather
//                            of the next forward) + clearing of the local gradient buffer.
//   signal / wait kernels    epoch flags in symmetric memory (st.release.sys / ld.acquire.sys).
//
// Replaces the reference's FSDP reduce_scatter_grads + per-shard optimizer + all-gather
// (src/fsdp.cpp:195-209,275-308,508-543), ZeRO (src/zero_optimizer_core.cpp:169-246,294-313), the
// 1-float gradient-norm all-reduce (src/fsdp.cpp:319-347, src/ddp.cpp:279-297) and the simulated
// DistributedContext collectives (src/distributed.cpp:26-100).
//
// Every wait on a peer is bounded (about one second, then an error code in *status and a normal
// return). Loads and stores to peers are ordinary global accesses: no TMA multicast anywhere.
#include "sm100_common.cuh"
#include "inv_api.h"

namespace inv {

constexpr int MAX_RANKS = 16;
constexpr uint64_t PEER_WAIT_NS = 1000000000ull;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until flags[r] >= epoch for every r < W. Returns false (and records the error) on timeout.
__device__ bool wait_all_flags(const uint32_t* flags, int W, uint32_t epoch, int* status, uint64_t limit_ns = PEER_WAIT_NS) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < W) {
    // tight polling; the (slow) global timer is read only every 256 polls
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
      if ((++spins & 0xffu) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > limit_ns) {
          s_ok = 0;
          if (status) atomicCAS(status, 0, ERR_WAIT_PEER);
          break;
        }
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// flags of every peer: peer p's word [rank] <- epoch
__global__ void signal_peers_kernel(PeerPtrs peer_flags, int W, int rank, uint32_t epoch) {
  __threadfence_system();
  if (threadIdx.x < W) st_release_sys(reinterpret_cast<uint32_t*>(peer_flags.p[threadIdx.x]) + rank, epoch);
}
__global__ void wait_flags_kernel(const uint32_t* flags, int W, uint32_t epoch, int* status, uint64_t limit_ns) {
  wait_all_flags(flags, W, epoch, status, limit_ns);
}

// Barrier over peer memory whose epoch lives on the device, so that it can sit inside a captured CUDA
// graph and advance on every replay: bump this rank's counter, publish it to every peer, wait until
// every peer has published a value at least as large.
__global__ void device_barrier_kernel(PeerPtrs peer_flags, uint32_t* local_flags, uint32_t* counter, int W, int rank, int* status) {
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) s_epoch = atomicAdd(counter, 1u) + 1u;
  __threadfence_system();
  __syncthreads();
  const uint32_t e = s_epoch;
  if (threadIdx.x < W) st_release_sys(reinterpret_cast<uint32_t*>(peer_flags.p[threadIdx.x]) + rank, e);
  wait_all_flags(local_flags, W, e, status);
}

// ------------------------------------------------------------------------------------------------
// Reduce-scatter. grads: peer pointers to the full fp32 gradient buffers. This rank owns [lo, lo+n).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fsdp_reduce_kernel(PeerPtrs grads, int W, int rank, long lo, long n, float* __restrict__ gshard,
                                                          float* __restrict__ sumsq_local, unsigned int* __restrict__ ticket,
                                                          const uint32_t* ready_flags, PeerPtrs norm_slots, PeerPtrs norm_flags,
                                                          uint32_t epoch, int* status) {
  if (ready_flags != nullptr && !wait_all_flags(ready_flags, W, epoch, status)) return;
  const long n4 = n / 4;
  float ss = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int r = 0; r < W; ++r) {
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(gshard)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __shared__ float red[8];
  __shared__ bool last;
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
    atomicAdd(sumsq_local, s);
    __threadfence();
    last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last) {
    // the last CTA publishes this rank's partial sum of squares to every peer, then raises the flag
    if (threadIdx.x < W) {
      const float total = atomicAdd(sumsq_local, 0.f);
      reinterpret_cast<float*>(norm_slots.p[threadIdx.x])[rank] = total;
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(norm_flags.p[threadIdx.x]) + rank, epoch);
    }
    if (threadIdx.x == 0) *ticket = 0;
  }
}

// ------------------------------------------------------------------------------------------------
// AdamW on the owned shard, fused with the parameter all-gather (push) and the gradient clear.
// hyper: see optim.cu (0 lr_adj, 1 beta1, 2 beta2, 3 eps, 4 lr*wd, 5 1/bias_corr2, 6 max_norm,
// 7 grad_scale, 8 decay_after). Elements at flat index >= decay_end get no weight decay.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void adamw_elem(float& p, float& m, float& v, float g, float lr_adj, float b1, float b2, float eps, float lrwd,
                                           float inv_bc2, bool decay_after) {
  if (!decay_after) p -= lrwd * p;
  m = b1 * m + (1.f - b1) * g;
  v = b2 * v + (1.f - b2) * g * g;
  p -= lr_adj * m / (sqrtf(v * inv_bc2) + eps);
  if (decay_after) p -= lrwd * p;
}

__global__ void __launch_bounds__(256) fsdp_adamw_push_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                                              const float* __restrict__ gshard, PeerPtrs params16, int W, int rank, long lo,
                                                              long n, long decay_end, const float* __restrict__ hyper,
                                                              const float* norm_slots_local, const uint32_t* norm_flags_local,
                                                              float* __restrict__ local_grads, long total, float* sumsq_local,
                                                              unsigned int* ticket, PeerPtrs done_flags, uint32_t epoch, int* status) {
  if (!wait_all_flags(norm_flags_local, W, epoch, status)) return;
  float norm_sq = 0.f;
  for (int r = 0; r < W; ++r) norm_sq += norm_slots_local[r];
  const float lr_adj = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], lrwd = hyper[4], inv_bc2 = hyper[5];
  const float max_norm = hyper[6];
  float gs = hyper[7];
  const bool decay_after = hyper[8] != 0.f;
  if (max_norm > 0.f) gs *= fminf(1.f, max_norm / (sqrtf(norm_sq) * gs + 1e-6f));
  const long n4 = n / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(master)[i], mv = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
    const float4 gv = reinterpret_cast<const float4*>(gshard)[i];
    const float wd = (lo + i * 4 < decay_end) ? lrwd : 0.f;
    adamw_elem(pv.x, mv.x, vv.x, gv.x * gs, lr_adj, b1, b2, eps, wd, inv_bc2, decay_after);
    adamw_elem(pv.y, mv.y, vv.y, gv.y * gs, lr_adj, b1, b2, eps, wd, inv_bc2, decay_after);
    adamw_elem(pv.z, mv.z, vv.z, gv.z * gs, lr_adj, b1, b2, eps, wd, inv_bc2, decay_after);
    adamw_elem(pv.w, mv.w, vv.w, gv.w * gs, lr_adj, b1, b2, eps, wd, inv_bc2, decay_after);
    reinterpret_cast<float4*>(master)[i] = pv;
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    uint2 o;
    o.x = pack_bf16x2(pv.x, pv.y);
    o.y = pack_bf16x2(pv.z, pv.w);
    // all-gather by pushing: own copy first, then every peer
    for (int k = 0; k < W; ++k) {
      const int r = (rank + k) % W;
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(params16.p[r]) + lo)[i] = o;
    }
  }
  // every peer has finished reading this rank's gradients (their norm flags arrived): clear them
  const long t4 = total / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < t4; i += (long)gridDim.x * blockDim.x)
    reinterpret_cast<float4*>(local_grads)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  __shared__ bool last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) {
      *ticket = 0;
      *sumsq_local = 0.f;
    }
    __threadfence_system();
    if (threadIdx.x < W) st_release_sys(reinterpret_cast<uint32_t*>(done_flags.p[threadIdx.x]) + rank, epoch);
  }
}

// Plain P2P all-gather (pull): out[r*n .. ] <- peer r's src[0..n). Used for shard gathers outside the step.
__global__ void allgather_pull_kernel(PeerPtrs src, int W, long n16, uint4* __restrict__ out) {
  for (int r = 0; r < W; ++r) {
    const uint4* s = reinterpret_cast<const uint4*>(src.p[r]);
    uint4* d = out + (long)r * n16;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n16; i += (long)gridDim.x * blockDim.x) d[i] = s[i];
  }
}

// All-reduce (sum) of fp32 vectors over peer memory, two-shot: each rank reduces its slice from all
// peers and writes the result into every peer's buffer. In-place on the symmetric buffers.
__global__ void allreduce_twoshot_kernel(PeerPtrs bufs, int W, int rank, long n4) {
  const long per = (n4 + W - 1) / W;
  const long lo = (long)rank * per;
  const long hi = lo + per < n4 ? lo + per : n4;
  for (long i = lo + blockIdx.x * (long)blockDim.x + threadIdx.x; i < hi; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < W; ++r) {
      const float4 v = reinterpret_cast<const float4*>(bufs.p[r])[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    for (int k = 0; k < W; ++k) reinterpret_cast<float4*>(bufs.p[(rank + k) % W])[i] = acc;
  }
}

// ---- stand-alone collectives through the switch (NVLS) ----
// `mc` is the multicast address of a symmetric buffer: a load-reduce on it returns the sum over all
// ranks' copies (added inside the switch), a store on it lands in every rank's copy. Each rank handles
// 1/W of the vector, so every element crosses this GPU's links once in each direction.
__device__ __forceinline__ float4 mc_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_f32x4(float* mc_addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// In-place all-reduce (sum, optionally scaled) of n4 float4 on the symmetric buffer behind `mc`.
__global__ void nvls_allreduce_kernel(float* mc, int W, int rank, long n4, float scale) {
  const long per = (n4 + W - 1) / W;
  const long lo = (long)rank * per, hi = lo + per < n4 ? lo + per : n4;
  for (long i = lo + blockIdx.x * (long)blockDim.x + threadIdx.x; i < hi; i += (long)gridDim.x * blockDim.x) {
    float4 v = mc_ld_reduce_f32x4(mc + i * 4);
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    mc_st_f32x4(mc + i * 4, v);
  }
}
// out[0..per4) = sum over ranks of their buffer[rank*per4 ..]; the symmetric buffer is left untouched.
__global__ void nvls_reduce_scatter_kernel(const float* mc, float* __restrict__ out, int rank, long per4) {
  const float* base = mc + (long)rank * per4 * 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < per4; i += (long)gridDim.x * blockDim.x)
    reinterpret_cast<float4*>(out)[i] = mc_ld_reduce_f32x4(base + i * 4);
}
// every rank's buffer[rank*per4 ..] <- this rank's src[0..per4)
__global__ void nvls_allgather_kernel(float* mc, const float* __restrict__ src, int rank, long per4) {
  float* base = mc + (long)rank * per4 * 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < per4; i += (long)gridDim.x * blockDim.x)
    mc_st_f32x4(base + i * 4, reinterpret_cast<const float4*>(src)[i]);
}
// Reduce-scatter over plain peer loads: out = sum_r peer_r[rank*per4 ..].
__global__ void p2p_reduce_scatter_kernel(PeerPtrs bufs, int W, int rank, long per4, float* __restrict__ out) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < per4; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < W; ++k) {
      const float4 v = reinterpret_cast<const float4*>(bufs.p[(rank + k) % W])[(long)rank * per4 + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(out)[i] = acc;
  }
}
// All-to-all (pull): out[r*chunk16 ..] <- peer r's src[rank*chunk16 ..], 16-byte units.
__global__ void alltoall_pull_kernel(PeerPtrs src, int W, int rank, long chunk16, uint4* __restrict__ out) {
  for (int k = 0; k < W; ++k) {
    const int r = (rank + k) % W;
    const uint4* s = reinterpret_cast<const uint4*>(src.p[r]) + (long)rank * chunk16;
    uint4* d = out + (long)r * chunk16;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < chunk16; i += (long)gridDim.x * blockDim.x) d[i] = s[i];
  }
}

static int fill_ptrs(PeerPtrs& pp, const uint64_t* host_ptrs, int W) {
  if (W < 1 || W > MAX_RANKS) return -ERR_BAD_ARG;
  for (int i = 0; i < MAX_RANKS; ++i) pp.p[i] = i < W ? reinterpret_cast<void*>(host_ptrs[i]) : nullptr;
  return 0;
}

}  // namespace inv

using namespace inv;
#define RET_LAUNCH()                        \
  do {                                      \
    cudaError_t e = cudaGetLastError();     \
    return e == cudaSuccess ? 0 : -(int)e;  \
  } while (0)

// peer_flags: host array of W device pointers (each rank's flag array, W words).
extern "C" int inv_signal_peers(const uint64_t* peer_flags, int W, int rank, uint32_t epoch, void* stream) {
  PeerPtrs pf;
  if (fill_ptrs(pf, peer_flags, W)) return -ERR_BAD_ARG;
  signal_peers_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pf, W, rank, epoch);
  RET_LAUNCH();
}
extern "C" int inv_wait_flags(const void* flags, int W, uint32_t epoch, int* status, void* stream) {
  if (W < 1 || W > MAX_RANKS) return -ERR_BAD_ARG;
  wait_flags_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const uint32_t*)flags, W, epoch, status, PEER_WAIT_NS);
  RET_LAUNCH();
}
// The same wait with the caller's time limit (nanoseconds of the global timer): after it the kernel writes ERR_WAIT_PEER to
// *status and returns normally, so the context stays usable. Used to exercise the error path without hanging anything.
extern "C" int inv_wait_flags_limit(const void* flags, int W, uint32_t epoch, long limit_ns, int* status, void* stream) {
  if (W < 1 || W > MAX_RANKS || limit_ns < 0) return -ERR_BAD_ARG;
  wait_flags_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const uint32_t*)flags, W, epoch, status, (uint64_t)limit_ns);
  RET_LAUNCH();
}

extern "C" int inv_fsdp_reduce(const uint64_t* peer_grads, int W, int rank, long lo, long n, float* gshard, float* sumsq_local,
                               unsigned int* ticket, const void* ready_flags, const uint64_t* peer_norm_slots,
                               const uint64_t* peer_norm_flags, uint32_t epoch, int* status, void* stream) {
  if (n % 4 || lo % 4) return -ERR_BAD_ARG;
  PeerPtrs g, ns, nf;
  if (fill_ptrs(g, peer_grads, W) || fill_ptrs(ns, peer_norm_slots, W) || fill_ptrs(nf, peer_norm_flags, W)) return -ERR_BAD_ARG;
  fsdp_reduce_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>(g, W, rank, lo, n, gshard, sumsq_local, ticket, (const uint32_t*)ready_flags, ns,
                                                                nf, epoch, status);
  RET_LAUNCH();
}

extern "C" int inv_fsdp_adamw_push(float* master, float* m, float* v, const float* gshard, const uint64_t* peer_params16, int W, int rank,
                                   long lo, long n, long decay_end, const float* hyper, const float* norm_slots_local,
                                   const void* norm_flags_local, float* local_grads, long total, float* sumsq_local, unsigned int* ticket,
                                   const uint64_t* peer_done_flags, uint32_t epoch, int* status, void* stream) {
  if (n % 4 || lo % 4 || total % 4 || decay_end % 4) return -ERR_BAD_ARG;
  PeerPtrs pp, df;
  if (fill_ptrs(pp, peer_params16, W) || fill_ptrs(df, peer_done_flags, W)) return -ERR_BAD_ARG;
  fsdp_adamw_push_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>(master, m, v, gshard, pp, W, rank, lo, n, decay_end, hyper, norm_slots_local,
                                                                    (const uint32_t*)norm_flags_local, local_grads, total, sumsq_local, ticket, df,
                                                                    epoch, status);
  RET_LAUNCH();
}

extern "C" int inv_allgather_pull(const uint64_t* peer_src, int W, long nbytes, void* out, void* stream) {
  if (nbytes % 16) return -ERR_BAD_ARG;
  PeerPtrs s;
  if (fill_ptrs(s, peer_src, W)) return -ERR_BAD_ARG;
  allgather_pull_kernel<<<148 * 2, 256, 0, (cudaStream_t)stream>>>(s, W, nbytes / 16, (uint4*)out);
  RET_LAUNCH();
}

extern "C" int inv_allreduce_f32(const uint64_t* peer_bufs, int W, int rank, long n, void* stream) {
  if (n % 4) return -ERR_BAD_ARG;
  PeerPtrs b;
  if (fill_ptrs(b, peer_bufs, W)) return -ERR_BAD_ARG;
  allreduce_twoshot_kernel<<<148 * 2, 256, 0, (cudaStream_t)stream>>>(b, W, rank, n / 4);
  RET_LAUNCH();
}

// counter: one device word per flag set, starts at 0 on every rank.
extern "C" int inv_device_barrier(const uint64_t* peer_flags, void* local_flags, void* counter, int W, int rank, int* status, void* stream) {
  PeerPtrs pf;
  if (fill_ptrs(pf, peer_flags, W)) return -ERR_BAD_ARG;
  device_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pf, (uint32_t*)local_flags, (uint32_t*)counter, W, rank, status);
  RET_LAUNCH();
}

// The callers bracket these with a device barrier over the peer flags: all ranks' inputs must be in place
// before a kernel reads them, and nobody may overwrite a buffer until every rank has finished reading it.
extern "C" int inv_nvls_allreduce_f32(void* mc_ptr, int W, int rank, long n, float scale, void* stream) {
  if (n % 4 || W < 1 || !mc_ptr) return -ERR_BAD_ARG;
  nvls_allreduce_kernel<<<148 * 2, 256, 0, (cudaStream_t)stream>>>((float*)mc_ptr, W, rank, n / 4, scale);
  RET_LAUNCH();
}
extern "C" int inv_nvls_reduce_scatter_f32(const void* mc_ptr, float* out, int rank, long per, void* stream) {
  if (per % 4 || !mc_ptr) return -ERR_BAD_ARG;
  nvls_reduce_scatter_kernel<<<148 * 2, 256, 0, (cudaStream_t)stream>>>((const float*)mc_ptr, out, rank, per / 4);
  RET_LAUNCH();
}
extern "C" int inv_nvls_allgather_f32(void* mc_ptr, const float* src, int rank, long per, void* stream) {
  if (per % 4 || !mc_ptr) return -ERR_BAD_ARG;
  nvls_allgather_kernel<<<148 * 2, 256, 0, (cudaStream_t)stream>>>((float*)mc_ptr, src, rank, per / 4);
  RET_LAUNCH();
}
extern "C" int inv_p2p_reduce_scatter_f32(const uint64_t* peer_bufs, int W, int rank, long per, float* out, void* stream) {
  if (per % 4) return -ERR_BAD_ARG;
  PeerPtrs b;
  if (fill_ptrs(b, peer_bufs, W)) return -ERR_BAD_ARG;
  p2p_reduce_scatter_kernel<<<148 * 2, 256, 0, (cudaStream_t)stream>>>(b, W, rank, per / 4, out);
  RET_LAUNCH();
}
extern "C" int inv_alltoall_pull(const uint64_t* peer_src, int W, int rank, long chunk_bytes, void* out, void* stream) {
  if (chunk_bytes % 16) return -ERR_BAD_ARG;
  PeerPtrs s;
  if (fill_ptrs(s, peer_src, W)) return -ERR_BAD_ARG;
  alltoall_pull_kernel<<<148 * 2, 256, 0, (cudaStream_t)stream>>>(s, W, rank, chunk_bytes / 16, (uint4*)out);
  RET_LAUNCH();
}
