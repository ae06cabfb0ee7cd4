// Kernel-map construction on the GPU: the step right before the convolution path.
//
// The reference never builds kernel maps (it loads them from files, spconv-test.py:63-73); every
// caller of the operator needs them.  These builders produce the canonical form the rest of this
// library documents — offset-major, ascending output row inside an offset, offsets enumerated
// lexicographically over (dx, dy, dz) — bit-identical to the host builder in fgms_b200/maps.py.
//
// Common scheme: a dense table T[k][o] (k_vol rows, one column per output voxel) receives the input
// row of pair (k, o) or -1; a device-wide exclusive scan of "T != -1" over the table in row-major order
// is exactly the position of every pair in the canonical flat arrays, and its value at the start of
// row k is kpos[k].
//   submanifold : hash table coordinate -> row; T[k][o] = lookup(coords[o] + d_k)
//   strided     : parents = floor(coords / s); unique parents (hash set), sorted (cub radix sort) = the
//                 output voxels; T[offset of i][parent row of i] = i
//   transposed  : T[k][in_map[j]] = out_map[j] for the pairs j of offset k
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"

namespace fgms {
namespace maps {

constexpr int COORD_BITS = 21;
constexpr int COORD_BIAS = 1 << 20;  // coordinates in [-2^20, 2^20) pack into 21 bits each
constexpr unsigned long long EMPTY_KEY = ~0ull;
constexpr int SCAN_THREADS = 512;
constexpr int SCAN_ITEMS = 8;  // table entries per thread
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

__device__ __forceinline__ bool pack(int x, int y, int z, unsigned long long* key) {
  const unsigned ux = (unsigned)(x + COORD_BIAS), uy = (unsigned)(y + COORD_BIAS), uz = (unsigned)(z + COORD_BIAS);
  if ((ux | uy | uz) >> COORD_BITS) return false;
  *key = ((unsigned long long)ux << (2 * COORD_BITS)) | ((unsigned long long)uy << COORD_BITS) | uz;
  return true;
}
__device__ __forceinline__ void unpack(unsigned long long key, int* x, int* y, int* z) {
  const unsigned m = (1u << COORD_BITS) - 1;
  *x = (int)((key >> (2 * COORD_BITS)) & m) - COORD_BIAS;
  *y = (int)((key >> COORD_BITS) & m) - COORD_BIAS;
  *z = (int)(key & m) - COORD_BIAS;
}
__device__ __forceinline__ unsigned slot_of(unsigned long long key, unsigned mask) {
  key ^= key >> 33;
  key *= 0xff51afd7ed558ccdull;
  key ^= key >> 33;
  key *= 0xc4ceb9fe1a85ec53ull;
  key ^= key >> 33;
  return (unsigned)key & mask;
}
__device__ __forceinline__ int floor_div(int a, int s) { return (a >= 0) ? a / s : -((-a + s - 1) / s); }

struct Table {
  unsigned long long* keys;  // [cap], EMPTY_KEY = free
  int* vals;                 // [cap]
  unsigned mask;             // cap - 1 (cap is a power of two, at least twice the entries)
};

// Returns the slot that holds `key` after the call; *fresh says whether this call put it there.
__device__ __forceinline__ int table_insert(const Table& t, unsigned long long key, bool* fresh) {
  unsigned h = slot_of(key, t.mask);
  for (unsigned probe = 0; probe <= t.mask; ++probe) {
    const unsigned long long old = atomicCAS(t.keys + h, EMPTY_KEY, key);
    if (old == EMPTY_KEY) { *fresh = true; return (int)h; }
    if (old == key) { *fresh = false; return (int)h; }
    h = (h + 1) & t.mask;
  }
  *fresh = false;
  return -1;  // table full: cannot happen with cap >= 2 n
}
__device__ __forceinline__ int table_find(const Table& t, unsigned long long key) {
  unsigned h = slot_of(key, t.mask);
  for (unsigned probe = 0; probe <= t.mask; ++probe) {
    const unsigned long long k = t.keys[h];
    if (k == key) return (int)h;
    if (k == EMPTY_KEY) return -1;
    h = (h + 1) & t.mask;
  }
  return -1;
}

// coordinate (or its parent under `stride`) of every voxel -> table.  value = row (stride 1; the values start
// at 0x7f7f7f7f).  A
// coordinate outside the packable range or met twice (stride 1) is counted as a problem.
__global__ void insert_kernel(const int32_t* __restrict__ coords, int n, int stride, Table t, int* n_unique) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int x = coords[3 * i], y = coords[3 * i + 1], z = coords[3 * i + 2];
  if (stride > 1) { x = floor_div(x, stride); y = floor_div(y, stride); z = floor_div(z, stride); }
  unsigned long long key;
  if (!pack(x, y, z, &key)) { report_problem(); return; }
  bool fresh;
  const int slot = table_insert(t, key, &fresh);
  if (slot < 0) { report_problem(); return; }
  if (stride == 1) {
    atomicMin(t.vals + slot, i);     // a voxel met twice keeps its first row, whichever thread got here first
    if (!fresh) report_problem();    // duplicate voxel
  } else if (fresh) {
    atomicAdd(n_unique, 1);
  }
}

// T[k][o] = row of coords[o] + d_k, or -1
__global__ void submanifold_fill_kernel(const int32_t* __restrict__ coords, int n, int ks, Table t, int* __restrict__ dense) {
  const long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long total = (long long)ks * ks * ks * n;
  if (j >= total) return;
  const int k = (int)(j / n), o = (int)(j % n);
  const int r = ks / 2;
  const int dx = k / (ks * ks) - r, dy = (k / ks) % ks - r, dz = k % ks - r;
  unsigned long long key;
  int src = -1;
  if (pack(coords[3 * o] + dx, coords[3 * o + 1] + dy, coords[3 * o + 2] + dz, &key)) {
    const int slot = table_find(t, key);
    if (slot >= 0) src = t.vals[slot];
  }
  dense[j] = src;
}

// occupied slots -> list of keys (any order)
__global__ void collect_keys_kernel(Table t, unsigned long long* __restrict__ out, int* counter) {
  const unsigned h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h > t.mask) return;
  const unsigned long long k = t.keys[h];
  if (k != EMPTY_KEY) out[atomicAdd(counter, 1)] = k;
}

// sorted unique parents: their coordinates, and their rank as the table value
__global__ void rank_kernel(const unsigned long long* __restrict__ sorted, int n_out, Table t, int32_t* __restrict__ out_coords) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_out) return;
  const unsigned long long key = sorted[r];
  const int slot = table_find(t, key);
  if (slot >= 0) t.vals[slot] = r; else report_problem();
  int x, y, z;
  unpack(key, &x, &y, &z);
  out_coords[3 * r] = x; out_coords[3 * r + 1] = y; out_coords[3 * r + 2] = z;
}

// T[offset of i][parent row of i] = i
__global__ void strided_fill_kernel(const int32_t* __restrict__ coords, int n, int stride, int n_out, Table t, int* __restrict__ dense) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int x = coords[3 * i], y = coords[3 * i + 1], z = coords[3 * i + 2];
  const int px = floor_div(x, stride), py = floor_div(y, stride), pz = floor_div(z, stride);
  unsigned long long key;
  if (!pack(px, py, pz, &key)) return;  // already counted by insert_kernel
  const int slot = table_find(t, key);
  if (slot < 0) { report_problem(); return; }
  const int o = t.vals[slot];
  const int k = ((x - px * stride) * stride + (y - py * stride)) * stride + (z - pz * stride);
  dense[(size_t)k * n_out + o] = i;
}

// T[k][in_map[j]] = out_map[j]
__global__ void transpose_fill_kernel(const int32_t* __restrict__ kpos, const int32_t* __restrict__ in_map,
                                      const int32_t* __restrict__ out_map, int k_vol, long long pairs, int n_cols,
                                      int* __restrict__ dense) {
  const long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (j >= pairs) return;
  int lo = 0, hi = k_vol;  // offset of pair j: kpos[lo] <= j < kpos[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(kpos + mid) <= j) lo = mid; else hi = mid;
  }
  const int c = in_map[j];
  if (c < 0 || c >= n_cols) { report_problem(); return; }
  dense[(size_t)lo * n_cols + c] = out_map[j];
}

__global__ void fill_kernel(int* __restrict__ p, long long count, int v) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) p[i] = v;
}

// ---- exclusive scan of (dense != -1) in three kernels, fused with the compaction -------------------
__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {  // SCAN_THREADS threads
  __shared__ int warp_sums[SCAN_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < SCAN_THREADS / 32 ? warp_sums[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    if (lane < SCAN_THREADS / 32) warp_sums[lane] = w;  // inclusive sums of the warps
  }
  __syncthreads();
  const int before = warp ? warp_sums[warp - 1] : 0;
  *total = warp_sums[SCAN_THREADS / 32 - 1];
  __syncthreads();
  return before + incl - v;
}

__global__ void __launch_bounds__(SCAN_THREADS) tile_count_kernel(const int* __restrict__ dense, long long total, int* __restrict__ tile_sums) {
  const long long base = (long long)blockIdx.x * SCAN_TILE + (long long)threadIdx.x * SCAN_ITEMS;
  int c = 0;
#pragma unroll
  for (int u = 0; u < SCAN_ITEMS; ++u)
    if (base + u < total && dense[base + u] >= 0) ++c;
  int sum;
  block_exclusive_scan(c, &sum);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = sum;
}

// one block: exclusive scan of the tile sums in place; the grand total goes to kpos[k_vol]
__global__ void __launch_bounds__(SCAN_THREADS) tile_scan_kernel(int* __restrict__ tile_sums, int n_tiles, int32_t* __restrict__ kpos, int k_vol) {
  int carry = 0;
  for (int b0 = 0; b0 < n_tiles; b0 += SCAN_THREADS) {
    const int i = b0 + threadIdx.x;
    const int v = i < n_tiles ? tile_sums[i] : 0;
    int sum;
    const int ex = block_exclusive_scan(v, &sum);
    if (i < n_tiles) tile_sums[i] = carry + ex;
    carry += sum;
  }
  if (threadIdx.x == 0) kpos[k_vol] = carry;
}

__global__ void __launch_bounds__(SCAN_THREADS) compact_kernel(const int* __restrict__ dense, long long total, int n_cols,
                                                               const int* __restrict__ tile_sums, int32_t* __restrict__ in_map,
                                                               int32_t* __restrict__ out_map, int32_t* __restrict__ kpos) {
  const long long base = (long long)blockIdx.x * SCAN_TILE + (long long)threadIdx.x * SCAN_ITEMS;
  int v[SCAN_ITEMS];
  int c = 0;
#pragma unroll
  for (int u = 0; u < SCAN_ITEMS; ++u) {
    v[u] = base + u < total ? dense[base + u] : -1;
    if (v[u] >= 0) ++c;
  }
  int sum;
  int pos = tile_sums[blockIdx.x] + block_exclusive_scan(c, &sum);
#pragma unroll
  for (int u = 0; u < SCAN_ITEMS; ++u) {
    const long long j = base + u;
    if (j < total) {
      const int col = (int)(j % n_cols);
      if (col == 0) kpos[j / n_cols] = pos;  // pairs before the first column of this offset
      if (v[u] >= 0) {
        in_map[pos] = v[u];
        out_map[pos] = col;
        ++pos;
      }
    }
  }
}

// ---- host side: workspace layout and the shared scan + compaction step -----------------------------
inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
inline unsigned table_capacity(int n) {
  unsigned cap = 64;
  while (cap < 2u * (unsigned)(n > 0 ? n : 1)) cap <<= 1;
  return cap;
}

struct Layout {  // offsets into the caller's workspace
  size_t keys, vals, dense, tile_sums, counter, ukeys, ukeys_sorted, cub, total;
  size_t cub_bytes;
  unsigned cap;
};
// n = voxels whose coordinates go into the table, n_cols = columns of the dense table
inline Layout layout(int n, int n_cols, int k_vol) {
  Layout L;
  L.cap = table_capacity(n);
  const long long cells = (long long)k_vol * (n_cols > 0 ? n_cols : 1);
  const long long tiles = (cells + SCAN_TILE - 1) / SCAN_TILE;
  const size_t nn = (size_t)(n > 0 ? n : 1);
  size_t off = 0;
  L.keys = off; off += align256((size_t)L.cap * 8);
  L.vals = off; off += align256((size_t)L.cap * 4);
  L.dense = off; off += align256((size_t)cells * 4);
  L.tile_sums = off; off += align256((size_t)tiles * 4);
  L.counter = off; off += 256;
  L.ukeys = off; off += align256(nn * 8);
  L.ukeys_sorted = off; off += align256(nn * 8);
  L.cub_bytes = 0;
  cub::DeviceRadixSort::SortKeys(nullptr, L.cub_bytes, (const unsigned long long*)nullptr, (unsigned long long*)nullptr,
                                 (int)nn, 0, 3 * COORD_BITS);
  L.cub = off; off += align256(L.cub_bytes);
  L.total = off;
  return L;
}

// scan + compaction of a filled dense table; false on a launch error
inline bool finish(const int* dense, int k_vol, int n_cols, int* tile_sums, int32_t* kpos, int32_t* in_map, int32_t* out_map,
                   cudaStream_t st) {
  const long long total = (long long)k_vol * n_cols;
  if (total == 0) return cudaMemsetAsync(kpos, 0, (size_t)(k_vol + 1) * 4, st) == cudaSuccess;
  const int tiles = (int)((total + SCAN_TILE - 1) / SCAN_TILE);
  tile_count_kernel<<<tiles, SCAN_THREADS, 0, st>>>(dense, total, tile_sums);
  tile_scan_kernel<<<1, SCAN_THREADS, 0, st>>>(tile_sums, tiles, kpos, k_vol);
  compact_kernel<<<tiles, SCAN_THREADS, 0, st>>>(dense, total, n_cols, tile_sums, in_map, out_map, kpos);
  return cudaGetLastError() == cudaSuccess;
}

}  // namespace maps
}  // namespace fgms
