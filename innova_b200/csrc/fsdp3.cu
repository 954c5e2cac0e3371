// Kernels of the fully sharded (stage 3) data-parallel engine that are not side jobs of a GEMM:
//
//   side_job_kernel          a gather / reduce side job (side_job.cuh) on its own, for the units that have no GEMM to ride in
//                            (the first unit of a step, whatever is still pending when the backward pass ends).
//   fsdp3_prepare_kernel     before a gradient buffer is reused: wait until every rank has finished pulling the previous
//                            contents ("consumed" flags), then clear it.
//   fsdp3_norm_kernel        global gradient norm: sum this rank's partial sums of squares in a fixed order, publish the
//                            total to every rank, wait for all of them, add them up in rank order.
//
// Reference behaviour covered: FullyShardedDataParallel stage 3 (src/fsdp.cpp:117-186 sharding, :188-227 gathers,
// :275-308 reduce-scatter + sharded step, :319-347 global-norm clip). Waits are bounded and report through *status.
#include "sm100_common.cuh"
#include "inv_api.h"
#include "side_job.cuh"

namespace inv {

__global__ void __launch_bounds__(320, 1) side_job_kernel(const SideJob job) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  run_side_job(job, (int)blockIdx.x, smem);
}

__global__ void __launch_bounds__(256) fsdp3_prepare_kernel(float4* __restrict__ buf, long n4, const uint32_t* consumed_flags, int W, int rank,
                                                            uint32_t epoch, int* status) {
  __shared__ int s_ok;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_ok = 1;
    s_abort = 0;
  }
  __syncthreads();
  if (consumed_flags != nullptr && threadIdx.x < W && threadIdx.x != rank) {
    if (!job_wait_flag(consumed_flags + threadIdx.x, epoch, &s_abort, status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) buf[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

struct NormPeers {
  float* slots[8];
  uint32_t* flags[8];
};

__global__ void __launch_bounds__(256) fsdp3_norm_kernel(const float* __restrict__ parts, int n_parts, NormPeers peers, const float* slots_local,
                                                         const uint32_t* flags_local, int W, int rank, uint32_t epoch, float* __restrict__ out,
                                                         int* status) {
  __shared__ int s_abort;
  __shared__ int s_ok;
  __shared__ float red[256];
  // fixed-shape sum of this rank's partial sums of squares: every thread a strided series, then a binary tree
  float s = 0.f;
  for (int i = threadIdx.x; i < n_parts; i += 256) s += parts[i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    s_abort = 0;
    s_ok = 1;
    for (int r = 0; r < W; ++r) peers.slots[r][rank] = red[0];
    __threadfence_system();
    for (int r = 0; r < W; ++r) job_st_release_sys(peers.flags[r] + rank, epoch);
  }
  __syncthreads();
  if ((int)threadIdx.x < W && !job_wait_flag(flags_local + threadIdx.x, epoch, &s_abort, status)) s_ok = 0;
  __syncthreads();
  if (threadIdx.x == 0 && s_ok) {
    float t = 0.f;
    for (int r = 0; r < W; ++r) t += reinterpret_cast<const volatile float*>(slots_local)[r];
    *out = t;
  }
}

}  // namespace inv

using namespace inv;

extern "C" int inv_side_job(const void* job, void* stream) {
  const SideJob* j = reinterpret_cast<const SideJob*>(job);
  if (j == nullptr || (j->kind != JOB_GATHER && j->kind != JOB_REDUCE) || j->W < 1 || j->W > 8 || j->n_ctas < 1 || (j->bytes & 15) ||
      (j->src_off & 15) || (j->dst_stride & 15) || (reinterpret_cast<uintptr_t>(j->dst) & 15))
    return -ERR_BAD_ARG;
  static bool configured = false;
  const int smem = SIDE_JOB_SMEM + 128;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(side_job_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  side_job_kernel<<<j->n_ctas, 320, smem, (cudaStream_t)stream>>>(*j);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

extern "C" int inv_side_job_struct_bytes() { return (int)sizeof(SideJob); }

extern "C" int inv_fsdp3_prepare(void* buf, long bytes, const uint32_t* consumed_flags, int W, int rank, uint32_t epoch, int* status,
                                 void* stream) {
  if ((bytes & 15) || (reinterpret_cast<uintptr_t>(buf) & 15)) return -ERR_BAD_ARG;
  if (bytes <= 0) return 0;
  long blocks = (bytes / 16 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  fsdp3_prepare_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<float4*>(buf), bytes / 16, consumed_flags, W, rank,
                                                                          epoch, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// slots / flags: per-rank addresses of a W-float exchange area and of a W-word flag set in symmetric memory.
extern "C" int inv_fsdp3_norm(const float* parts, int n_parts, const uint64_t* slot_ptrs, const uint64_t* flag_ptrs, int W, int rank,
                              uint32_t epoch, float* out, int* status, void* stream) {
  if (W < 1 || W > 8 || rank < 0 || rank >= W) return -ERR_BAD_ARG;
  NormPeers np;
  for (int r = 0; r < 8; ++r) {
    np.slots[r] = reinterpret_cast<float*>(slot_ptrs[r < W ? r : 0]);
    np.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r < W ? r : 0]);
  }
  fsdp3_norm_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(parts, n_parts, np, np.slots[rank], np.flags[rank], W, rank, epoch, out, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}
