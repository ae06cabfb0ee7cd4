// Thin wrappers over the sm_100a PTX this library uses: mbarriers, cp.async, the async-proxy
// fence, and tcgen05 (tensor-memory allocation, UMMA issue/commit, tensor-memory loads), plus the
// shared-memory and instruction descriptors of tcgen05.mma and the 128-byte-swizzled canonical
// operand layouts.  All waits are bounded: a wait that runs out returns false and the caller
// reports it instead of spinning forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fgms {
namespace umma {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One non-blocking probe of the barrier.  (mbarrier.try_wait may park the thread for an
// implementation-defined time slice and was measured to wake up late; hand-offs between the roles of
// these kernels are latency-critical, so the waiting lane probes with test_wait instead.)
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about one second of SM clock.  `abort_flag` (shared memory) lets one
// role tell the others to stop waiting once something has gone wrong.
constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (abort_flag && *abort_flag) return false;
      if (clock64() - start > WAIT_LIMIT_CYCLES) break;
    }
  }
  if (abort_flag) *abort_flag = 1;
  return false;
}

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while the kernel before
// it in the stream is still running.  griddep_wait() returns once that kernel has finished and its writes
// are visible: nothing it may have written (or may still read and this kernel overwrites) is touched
// before the call.  griddep_launch_dependents() lets the next such kernel in the stream start its own
// preamble as soon as this grid's CTAs make room.  Both do nothing in a kernel launched the plain way.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------ cp.async (16-byte, zero fill)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
// same with the number of bytes to read (16, or 0 for a zero-filled chunk) already in a register
__device__ __forceinline__ void cp_async16_n(uint32_t dst, const void* src, uint32_t n) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
// 4-byte copy (goes through L1): used to prefetch map entries into shared memory without tying up a register
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void st_shared_i32(uint32_t dst, int v) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_shared_i32(uint32_t src) {
  int v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(src) : "memory");
  return v;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// the mbarrier receives one arrival from this thread once all cp.async it has issued so far have landed
// (.noinc: the arrival counts against the barrier's expected count like an ordinary arrive)
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// make generic-proxy / cp.async writes to shared memory visible to the async proxy (tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------ tcgen05
// whole warp; ncols a power of two in [32, 512]; the base address lands in *smem_dst
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; one thread issues
template <bool TF32>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  if (TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
  }
}
// arrive on an mbarrier once every tcgen05.mma issued so far by this thread has finished
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32-bit, 16 consecutive columns: thread t of the warp reads lane (warp%4)*32 + t
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ descriptors
// Instruction descriptor of tcgen05.mma kind::f16 / kind::tf32 with fp32 accumulation:
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format  (0 = f16, 2 = tf32)
//   [15] A major  [16] B major (0 = K-major, 1 = MN-major)   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc(bool tf32, bool a_mn_major, bool b_mn_major, int m, int n) {
  return (1u << 4) | ((tf32 ? 2u : 0u) << 7) | ((tf32 ? 2u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle:
//   [0,14) start address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) version = 1 (sm_100)   [61,64) layout type = 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type = 2) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)layout_type << 61;
  return d;
}

// Canonical 128-byte-swizzled operand layouts (tile bases are 1024-byte aligned).
//
// K-major (the contraction index is contiguous in a row): a tile of R rows is stored as sub-tiles of
// [R rows x 128 bytes]; inside a sub-tile rows are 128 bytes apart, groups of 8 rows 1024 bytes apart
// (the stride byte offset), and the 16-byte chunk c of row r sits at chunk position c ^ (r % 8).
// One MMA consumes 32 bytes of every row: advancing the start address by 32 selects the next K step.
__host__ __device__ constexpr uint32_t kmajor_offset(uint32_t row, uint32_t byte_in_row, uint32_t rows) {
  return (byte_in_row >> 7) * (rows * 128u) + (row >> 3) * 1024u + (row & 7u) * 128u +
         ((((byte_in_row >> 4) & 7u) ^ (row & 7u)) << 4) + (byte_in_row & 15u);
}
// MN-major (the M or N index is contiguous in a row, one row per contraction index k): rows of
// [128 bytes] are grouped in atoms of 8 consecutive k (1024 bytes); atoms that follow each other in k
// are `sbo` bytes apart, atoms that follow each other along M/N (the next 128 bytes of every row) are
// `lbo` bytes apart; chunk c of row k sits at c ^ (k % 8).
__host__ __device__ constexpr uint32_t mnmajor_offset(uint32_t k, uint32_t byte_in_row, uint32_t lbo, uint32_t sbo) {
  return (byte_in_row >> 7) * lbo + (k >> 3) * sbo + (k & 7u) * 128u +
         ((((byte_in_row >> 4) & 7u) ^ (k & 7u)) << 4) + (byte_in_row & 15u);
}

// MN-major for 32-bit elements (tf32) has its own layout, "128-byte swizzle with 32-byte atomicity"
// (descriptor layout type 1): atoms are 4 consecutive k (512 bytes), and the 32-byte chunk q of row k
// sits at chunk position q ^ (k % 4).  `sbo` is the distance between atoms that follow each other in k.
__host__ __device__ constexpr uint32_t mnmajor32_offset(uint32_t k, uint32_t byte_in_row, uint32_t lbo, uint32_t sbo) {
  return (byte_in_row >> 7) * lbo + (k >> 2) * sbo + (k & 3u) * 128u +
         ((((byte_in_row >> 5) & 3u) ^ (k & 3u)) << 5) + (byte_in_row & 31u);
}

}  // namespace umma

// Launch with the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3((unsigned)grid);
  lc.blockDim = dim3((unsigned)block);
  lc.dynamicSmemBytes = smem;
  lc.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, kernel, static_cast<KArgs>(args)...);
}
}  // namespace fgms
