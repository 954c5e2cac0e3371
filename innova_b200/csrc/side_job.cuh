// Side jobs: the collective half of fully sharded data parallelism, run by a few helper CTAs that ride in the grid
// of a tensor-core GEMM (or in a small kernel of their own when no GEMM is at hand).
//
// The GEMM kernels here are persistent, one CTA per SM with nearly all of its shared memory, so a kernel on another
// stream gets no SM until the GEMM retires: a collective that should overlap compute has to be part of the compute
// kernel's own grid. A helper CTA owns no barriers or tensor memory of the GEMM; it drives the copy engine with bulk
// asynchronous copies (peer memory -> shared memory -> local memory, never with cluster multicast) and leaves.
//
//   JOB_GATHER  all-gather of one parameter unit: byte range [src_off, src_off + bytes) of every rank's shard buffer is
//               copied to dst + r * dst_stride. Peer r is read only after wait_flags[r] has reached wait_epoch
//               ("rank r's shards hold this step's parameters").
//   JOB_REDUCE  reduce-scatter of one gradient unit: this rank's slice [src_off, src_off + bytes) of every rank's fp32
//               gradient buffer is pulled through shared memory, summed in rank order, scaled and written (or added) to
//               the local fp32 shard `dst`; the sum of squares of the result goes to sumsq[cta]. Peer r is read only
//               after wait_flags[r] has reached wait_epoch ("rank r has finished this unit's backward"). When
//               signal_epoch != 0 the last helper CTA to finish writes it into word [rank] of every peer's
//               signal_flags ("this rank no longer reads your gradient buffer").
//
// Replaces the reference's FSDP allgather_param / reduce_scatter_grads loops (src/fsdp.cpp:188-227,275-308).
// Every wait is bounded and reports through *status.
#pragma once
#include "sm100_common.cuh"

namespace inv {

enum : int { JOB_NONE = 0, JOB_GATHER = 1, JOB_REDUCE = 2 };

struct SideJob {
  int kind;
  int W, rank, n_ctas;
  const void* src[8];
  long src_off;
  long bytes;
  void* dst;
  long dst_stride;
  const uint32_t* wait_flags;
  uint32_t wait_epoch;
  uint32_t signal_epoch;
  uint32_t* signal_flags[8];
  unsigned int* ticket;
  float* sumsq;
  float scale;
  int accumulate;
  int* status;
};

constexpr int SIDE_JOB_SMEM = 6 * 32768 + 64;  // ring of bulk-copy slots + barriers

__device__ __forceinline__ uint32_t job_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void job_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// One thread waits (at most about a second) for a peer's flag to reach the epoch.
__device__ __forceinline__ bool job_wait_flag(const uint32_t* flag, uint32_t epoch, volatile int* abort_flag, int* status) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while ((int32_t)(job_ld_acquire_sys(flag) - epoch) < 0) {
    if ((++spins & 0xffu) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > 1000000000ull) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, ERR_WAIT_PEER);
        return false;
      }
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");  // the bulk copies that follow read what the flag's writer published
  return true;
}
__device__ __forceinline__ void job_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---- all-gather of a parameter unit (one thread per helper CTA drives the copy engine) ----
static __device__ __noinline__ void job_gather(const SideJob& j, int cta, uint8_t* ring, uint64_t* bars, volatile int* abort_flag) {
  constexpr int SLOTS = 6, AHEAD = 4, CH = 32768;
  if (threadIdx.x >= 32) {
    // warps 1..: this rank's own shard, local memory to local memory with plain 16-byte accesses, this CTA's share of it
    const long n16 = j.bytes / 16;
    const long per = (n16 + j.n_ctas - 1) / j.n_ctas;
    const long lo = cta * per, hi = lo + per < n16 ? lo + per : n16;
    const uint4* s = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(j.src[j.rank]) + j.src_off);
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(j.dst) + j.rank * j.dst_stride);
    const long nt = blockDim.x - 32;
    long i = lo + (threadIdx.x - 32);
    for (; i + 3 * nt < hi; i += 4 * nt) {
      const uint4 a = s[i], b = s[i + nt], c = s[i + 2 * nt], e = s[i + 3 * nt];
      d[i] = a; d[i + nt] = b; d[i + 2 * nt] = c; d[i + 3 * nt] = e;
    }
    for (; i < hi; i += nt) d[i] = s[i];
    return;
  }
  if (threadIdx.x != 0) return;
  for (int s = 0; s < SLOTS; ++s) mbar_init(&bars[s], 1);
  *abort_flag = 0;
  fence_barrier_init();
  const long cpp = (j.bytes + CH - 1) / CH;  // chunks per peer
  const long total = cpp * (j.W - 1);        // the peers' shards only
  const long mine = cta < total ? (total - cta + j.n_ctas - 1) / j.n_ctas : 0;
  uint32_t gi = 0, gw = 0, ready = 0;
  auto chunk = [&](long i, int& r, long& off, uint32_t& bytes) {
    const long c = cta + i * j.n_ctas;
    r = (j.rank + 1 + (int)(c / cpp)) % j.W;  // nearest peer first
    off = (c % cpp) * CH;
    bytes = (uint32_t)(j.bytes - off < (long)CH ? j.bytes - off : (long)CH);
  };
  bool ok = true;
  for (long i = 0; ok && i < mine + AHEAD; ++i) {
    if (i < mine) {
      int r;
      long off;
      uint32_t bytes;
      chunk(i, r, off, bytes);
      if (!((ready >> r) & 1u)) {
        if (j.wait_flags != nullptr && !job_wait_flag(j.wait_flags + r, j.wait_epoch, abort_flag, j.status)) { ok = false; break; }
        ready |= 1u << r;
      }
      // the slot's previous store must have read its data: at most SLOTS - AHEAD - 1 newer stores may still be pending
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      const uint32_t slot = gi % SLOTS;
      mbar_expect_tx(&bars[slot], bytes);
      job_bulk_load(ring + slot * CH, reinterpret_cast<const uint8_t*>(j.src[r]) + j.src_off + off, bytes, &bars[slot]);
      ++gi;
    }
    if (i >= AHEAD) {
      int r;
      long off;
      uint32_t bytes;
      chunk(i - AHEAD, r, off, bytes);
      const uint32_t slot = gw % SLOTS;
      if (!mbar_wait(&bars[slot], (gw / SLOTS) & 1, abort_flag, j.status, ERR_WAIT_PEER)) { ok = false; break; }
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint8_t*>(j.dst) + r * j.dst_stride + off),
                   "r"(smem_u32(ring + slot * CH)), "r"(bytes)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      ++gw;
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (!ok) {  // give the loads still in flight a bounded time to land before the shared memory goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
}

// ---- reduce-scatter of a gradient unit (whole helper CTA) ----
static __device__ __noinline__ void job_reduce(const SideJob& j, int cta, uint8_t* ring, uint64_t* bars, volatile int* abort_flag) {
  // A chunk is CHB bytes from each of the W ranks; three 64 KB slots hold one chunk each, so that two chunks (128 KB, what
  // an NVLink round trip of a few microseconds needs to stay busy) are in flight while the third is summed.
  constexpr int SLOTS = 3;
  const int CHB = (65536 / j.W) & ~1023;
  __shared__ float red[32];
  __shared__ int s_ok;
  const int tid = threadIdx.x, nthr = blockDim.x;
  if (tid == 0) {
    for (int s = 0; s < SLOTS; ++s) mbar_init(&bars[s], 1);
    *abort_flag = 0;
    fence_barrier_init();
    int ok = 1;
    if (j.wait_flags != nullptr)
      for (int r = 0; ok && r < j.W; ++r)
        if (r != j.rank && !job_wait_flag(j.wait_flags + r, j.wait_epoch, abort_flag, j.status)) ok = 0;
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const long n_chunks = (j.bytes + CHB - 1) / CHB;
  const long mine = cta < n_chunks ? (n_chunks - cta + j.n_ctas - 1) / j.n_ctas : 0;
  auto issue = [&](long i) {  // thread 0: the W peers' pieces of my i-th chunk into slot i % SLOTS
    const long off = (cta + i * j.n_ctas) * (long)CHB;
    const uint32_t bytes = (uint32_t)(j.bytes - off < (long)CHB ? j.bytes - off : (long)CHB);
    const int slot = (int)(i % SLOTS);
    mbar_expect_tx(&bars[slot], bytes * j.W);
    for (int r = 0; r < j.W; ++r)
      job_bulk_load(ring + slot * 65536 + r * CHB, reinterpret_cast<const uint8_t*>(j.src[r]) + j.src_off + off, bytes, &bars[slot]);
  };
  if (tid == 0)
    for (long i = 0; i < SLOTS - 1 && i < mine; ++i) issue(i);
  float ss = 0.f;
  bool ok = true;
  for (long i = 0; i < mine; ++i) {
    if (tid == 0 && i + SLOTS - 1 < mine) issue(i + SLOTS - 1);  // its slot was read in iteration i - 1, behind the barrier below
    const int slot = (int)(i % SLOTS);
    if (!mbar_wait(&bars[slot], (uint32_t)(i / SLOTS) & 1, abort_flag, j.status, ERR_WAIT_PEER)) { ok = false; break; }
    const long off = (cta + i * j.n_ctas) * (long)CHB;
    const int n4 = (int)((j.bytes - off < (long)CHB ? j.bytes - off : (long)CHB) / 16);
    float4* out = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(j.dst) + off);
    for (int e = tid; e < n4; e += nthr) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < j.W; ++r) {
        const float4 v = reinterpret_cast<const float4*>(ring + slot * 65536 + r * CHB)[e];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      acc.x *= j.scale; acc.y *= j.scale; acc.z *= j.scale; acc.w *= j.scale;
      if (j.accumulate) {
        const float4 o = out[e];
        acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
      }
      out[e] = acc;
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
    __syncthreads();
  }
  if (!ok) {  // every thread leaves the loop at the same iteration (the abort flag is shared); let the loads in flight land
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    return;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int w = 0; w < (nthr + 31) / 32; ++w) s += red[w];
    if (j.sumsq != nullptr) j.sumsq[cta] = s;
    __threadfence_system();
    if (j.signal_epoch != 0 && atomicAdd(j.ticket, 1u) == (unsigned)j.n_ctas - 1) {
      *j.ticket = 0;
      for (int r = 0; r < j.W; ++r) job_st_release_sys(j.signal_flags[r] + j.rank, j.signal_epoch);
    }
  }
}

// Entry for a helper CTA: `smem` is at least SIDE_JOB_SMEM bytes, 128-byte aligned.
__device__ __forceinline__ void run_side_job(const SideJob& j, int cta, uint8_t* smem) {
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * 32768);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 6);
  if (j.kind == JOB_GATHER) job_gather(j, cta, smem, bars, abort_flag);
  else if (j.kind == JOB_REDUCE) job_reduce(j, cta, smem, bars, abort_flag);
}

}  // namespace inv
