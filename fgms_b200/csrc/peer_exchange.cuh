// Sum of the ranks' fp32 weight-gradient partial sums over peer memory (NVLink / NVSwitch), as one small kernel
// per rank that runs beside the input-gradient kernel.
//
// Every rank holds three peer-mapped buffers of the same size: `sums` (its own fp32 partial sums, written by its
// weight-gradient kernel), `reduced` (receives the total) and a few flag words.  The element range is cut into
// `world` slices; rank r owns slice r.  One call, on every rank:
//
//   1. announce   a thread stores this call's epoch into flag A[rank] of every rank (after a system-scope fence:
//                 the weight-gradient kernel before this one in the stream has finished, its sums are visible);
//   2. wait       until A[p] >= epoch for every p in this rank's own flags;
//   3. reduce     the rank's slice: load it from every rank's `sums` (plain peer loads, fixed order p = 0 .. world-1,
//                 so the total is the same bits on every run), add, store the total into every rank's `reduced`;
//   4. announce   the last CTA to finish stores the epoch into flag D[rank] of every rank;
//   5. wait       that same CTA waits until D[p] >= epoch for every p: this rank's `reduced` is complete and no peer
//                 still reads its `sums`.  The other CTAs have left by then: a CTA that waited here would hold its
//                 place on an SM while the CTAs it waits for (its own rank's later ones included) may need one.
//
// The reference has no multi-GPU path (backend/spconv.cu has no collective); this replaces the NCCL all-reduce of
// the data-parallel step where its launch needs SMs the input-gradient kernel holds.  Only plain loads and stores
// cross the link: no multicast, no atomics on peer memory.  Every wait is bounded; one that runs out is counted
// (g_device_problems), the kernel returns, and the totals of that call are incomplete.  Epochs only grow, so flags
// are never cleared.  With epoch = 0 in the parameters the kernel numbers its calls itself (from the rank's CTA
// counter, which every call raises by the grid size), so that a launch can be replayed from a CUDA graph.
#pragma once

#include "common.cuh"

namespace fgms {

constexpr int PX_MAX_WORLD = 16;
constexpr int PX_THREADS = 128;  // small CTAs of few registers: they find room on SMs that a persistent kernel occupies
constexpr long long PX_WAIT_LIMIT_CYCLES = 2000000000ll;  // about one second of SM clock

struct PeerExchangeParams {
  const float* sums[PX_MAX_WORLD];   // every rank's partial sums (index = rank)
  float* reduced[PX_MAX_WORLD];      // every rank's buffer for the totals
  uint32_t* flags[PX_MAX_WORLD];     // every rank's flag words: A[0 .. world), D[world .. 2 world), then one CTA counter
  long long count;                   // fp32 values; a multiple of 4
  long long wait_limit;              // cycles a wait may take
  uint32_t epoch;                    // of this call: larger than that of any call before it; 0 = numbered on the device
  int rank, world;
};

__device__ __forceinline__ void px_store_flag(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t px_load_flag(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 px_load4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void px_store4(float* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Threads 0 .. world-1 of the CTA each watch one flag; the CTA learns whether all of them arrived in time.
__device__ __forceinline__ bool px_wait_all(const uint32_t* my_flags, int world, uint32_t epoch, long long limit) {
  __shared__ int timed_out;
  if (threadIdx.x == 0) timed_out = 0;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const long long start = clock64();
    // epochs are compared by their distance so that the counter may wrap
    while ((int32_t)(px_load_flag(my_flags + threadIdx.x) - epoch) < 0) {
      if (clock64() - start > limit) { timed_out = 1; break; }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return timed_out == 0;
}

// One 16-byte piece per thread and iteration: the loads of two ranks in flight, added in rank order as they
// arrive.  Few registers on purpose (see the launch bounds of the kernel).
__device__ __forceinline__ void px_reduce_slice(const PeerExchangeParams& p, long long first, long long hi, long long stride) {
  const int world = p.world;
  for (long long i = first; i < hi; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int q = 0;
    for (; q + 1 < world; q += 2) {
      const float4 a = px_load4(p.sums[q] + 4 * i);
      const float4 b = px_load4(p.sums[q + 1] + 4 * i);
      acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
      acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    }
    if (q < world) {
      const float4 a = px_load4(p.sums[q] + 4 * i);
      acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
    }
    for (int r = 0; r < world; ++r) px_store4(p.reduced[r] + 4 * i, acc);
  }
}

// At most 32 registers per thread (16 CTAs of 128 threads per SM by the bounds): the kernel is meant to run
// BESIDE the persistent forward / dgrad kernel, whose 17 warps leave the warp scheduler that holds five of them
// only 1024 free registers — room for exactly one warp of 32 registers per thread.  With more registers its CTAs
// are not scheduled until that kernel ends (measured: the exchange then starts when dgrad finishes).
__global__ void __launch_bounds__(PX_THREADS, 16) peer_exchange_kernel(PeerExchangeParams p) {
  const int world = p.world, rank = p.rank;
  uint32_t* mine = p.flags[rank];
  // Number of this call.  The CTA counter holds gridDim.x per finished call (the calls before this one have
  // finished: they were ahead in the stream) plus one per CTA of this call that is done already — fewer than
  // gridDim.x as long as this CTA is not: counter / gridDim.x is the number of calls before this one.
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) epoch_s = p.epoch != 0u ? p.epoch : *reinterpret_cast<volatile uint32_t*>(mine + 2 * world) / gridDim.x + 1u;
  __syncthreads();
  const uint32_t epoch = epoch_s;
  if (blockIdx.x == 0 && (int)threadIdx.x < world) {
    __threadfence_system();
    px_store_flag(p.flags[threadIdx.x] + rank, epoch);
  }
  bool ok = px_wait_all(mine, world, epoch, p.wait_limit);
  if (ok) {
    const long long n4 = p.count / 4;
    const long long lo = n4 * rank / world, hi = n4 * (rank + 1) / world;
    px_reduce_slice(p, lo + (long long)blockIdx.x * PX_THREADS + threadIdx.x, hi, (long long)gridDim.x * PX_THREADS);
  }
  // the last CTA of this rank to get here tells every rank that this rank's slice is written everywhere
  __shared__ int last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(mine + 2 * world, 1u) + 1u;
    __threadfence_system();  // what the other CTAs stored before they counted themselves is ordered before the flag below
    last = (done % gridDim.x) == 0;  // the counter is never cleared: every call adds gridDim.x
  }
  __syncthreads();
  if (last) {
    if ((int)threadIdx.x < world) px_store_flag(p.flags[threadIdx.x] + world + rank, epoch);
    if (ok) ok = px_wait_all(mine + world, world, epoch, p.wait_limit);
  }
  if (!ok && threadIdx.x == 0) report_problem();
}

}  // namespace fgms
