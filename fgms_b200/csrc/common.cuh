// Shared device-side pieces of the fgms_b200 kernels: the parameter block, the per-CTA tile
// table derived from `kpos`, bounds-checked map reads and the scatter-add primitives.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fgms {

// Number of problems kernels ran into (map entries out of range that were skipped, bounded
// waits that gave up).  Read and reset from the host through fgms_b200_device_status().
__device__ unsigned long long g_device_problems = 0ull;

__device__ __forceinline__ void report_problem() { atomicAdd(&g_device_problems, 1ull); }

// One gather -> GEMM -> scatter pass.  Forward and dgrad are the same pass with the two maps
// and the two channel counts exchanged and the weight matrix read transposed; the reference
// makes the same observation by passing its maps swapped (backend/spconv.cu:460).
struct GmsParams {
  const void* src;             // [n_gather , k_dim]  rows that are gathered
  const void* weights;         // [k_vol, c_in, c_out]
  void* dst;                   // [n_scatter, n_dim]  rows that are accumulated into
  const int32_t* kpos;         // [k_vol + 1]
  const int32_t* gather_map;   // [pairs]
  const int32_t* scatter_map;  // [pairs]
  int pairs;                   // entries the two maps hold: no position >= pairs is ever read
  int n_gather, n_scatter;
  int k_dim, n_dim;            // contraction width, output width
  int c_in, c_out;             // layout of `weights`
  int k_vol;
  int dense_rows;              // > 0: one more segment of `dense_rows` identity pairs ...
  int dense_weight;            // ... that uses this weight index (the "separate mid" term)
};

struct WgradParams {
  const void* feats;     // [n_in , c_in ]
  const void* out_grad;  // [n_out, c_out]
  float* dw;             // [k_vol, c_in, c_out] fp32 accumulator
  const int32_t* kpos;
  const int32_t* in_map;
  const int32_t* out_map;
  int pairs;  // entries the two maps hold
  int n_in, n_out, c_in, c_out, k_vol;
  // fp16 storage, tensor-core kernel only: add every CTA's fp32 partial sums, rounded to fp16, straight
  // into the fp16 gradient (dw is then unused)
  __half* dw_f16 = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Tile table.  Segment s < k_vol holds the pairs kpos[s] .. kpos[s+1] of kernel offset s; the
// optional last segment holds the identity pairs of the dense centre term.  Every segment is cut
// into tiles of TILE pairs that never straddle two segments — the property the reference gets by
// padding each offset to a multiple of 256 rows on the host (kpos_quantized, cpu-check.py:6-14)
// and searching the padded prefix sums per block (backend/utils.cuh:6-27).  Here each CTA derives
// the table from the unpadded `kpos` itself, so no padded rows are ever scheduled.
// ---------------------------------------------------------------------------------------------
// `kpos` comes from the caller's device memory and is not trusted: every entry is clamped to
// [0, pairs] (pairs = length of the maps) on its way into shared memory, so a stale or mismatched
// kpos can shorten segments but never moves a map read past the end of the maps.  A clamped entry
// is counted as a problem once per launch.
__device__ __forceinline__ void build_tile_table(int TILE, const int32_t* __restrict__ kpos, int pairs, int k_vol,
                                                 int dense_rows, int* kpos_s /* [k_vol+1] */,
                                                 int* tile_start /* [k_vol+2] */) {
  for (int s = threadIdx.x; s <= k_vol; s += blockDim.x) {
    const int v = __ldg(kpos + s);
    const int c = min(max(v, 0), pairs);
    if (v != c && blockIdx.x == 0) report_problem();
    kpos_s[s] = c;
  }
  __syncthreads();
  // counts first (parallel), then the first warp turns them into running sums, 32 segments at a time
  for (int s = threadIdx.x; s <= k_vol; s += blockDim.x) {
    int cnt = (s < k_vol) ? (kpos_s[s + 1] - kpos_s[s]) : dense_rows;
    if (cnt < 0) cnt = 0;
    tile_start[s + 1] = (cnt + TILE - 1) / TILE;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int carry = 0;
    for (int s0 = 0; s0 <= k_vol; s0 += 32) {
      const int s = s0 + lane;
      int v = s <= k_vol ? tile_start[s + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      if (s <= k_vol) tile_start[s + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) tile_start[0] = 0;
  }
  __syncthreads();
}

// Segment that owns tile t (tile_start is non-decreasing; empty segments are skipped).
__device__ __forceinline__ int find_segment(const int* tile_start, int n_seg, int t) {
  int lo = 0, hi = n_seg;  // invariant: tile_start[lo] <= t < tile_start[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (tile_start[mid] <= t) lo = mid; else hi = mid;
  }
  return lo;
}

// Contiguous share of `total` tiles for this CTA.
__device__ __forceinline__ void cta_tile_range(int total, int* t0, int* t1) {
  long long g = gridDim.x, b = blockIdx.x;
  *t0 = (int)((long long)total * b / g);
  *t1 = (int)((long long)total * (b + 1) / g);
}

// ---------------------------------------------------------------------------------------------
// element helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

__device__ __forceinline__ void red_add(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void red_add(__half* p, float v) { atomicAdd(p, __float2half_rn(v)); }

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void red_add_h8(__half* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

__device__ __forceinline__ void red_add_h4(__half* p, uint32_t a, uint32_t b) {
  asm volatile("red.global.add.noftz.v2.f16x2 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// Add v[0..n) to consecutive elements starting at p.  `vec` says that p is suitably aligned for one
// vector red of N elements (16 bytes for four floats, 8 bytes for four halves) — decided once per
// launch from the channel count and the base address.
template <int N>
__device__ __forceinline__ void scatter_add(float* p, const float (&v)[N], int valid, bool vec) {
  if constexpr (N == 4) {
    if (vec && valid == 4) {
      red_add_v4(p, v[0], v[1], v[2], v[3]);
      return;
    }
  }
  {
#pragma unroll
    for (int c = 0; c < N; ++c)
      if (c < valid) red_add(p + c, v[c]);
  }
}
template <int N>
__device__ __forceinline__ void scatter_add(__half* p, const float (&v)[N], int valid, bool vec) {
  if constexpr (N == 4) {
    if (vec && valid == 4) {
      red_add_h4(p, pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
      return;
    }
  }
  {
#pragma unroll
    for (int c = 0; c < N; ++c)
      if (c < valid) red_add(p + c, v[c]);
  }
}

}  // namespace fgms
