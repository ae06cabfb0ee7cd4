// Tensor-core kernels for sm_100a: gather -> tcgen05.mma (accumulators in tensor memory) -> scatter.
//
// Both kernels are persistent (one CTA per SM, each walking a contiguous share of the tile list
// derived from `kpos`) and warp-specialised:
//
//   warps 0-3  drain      tcgen05.ld of the fp32 accumulators, conversion to the storage type, parked in a
//                         swizzled shared-memory patch (wgrad: straight to vector red.global.add.f32)
//   warp  4    MMA        one thread issues tcgen05.mma / tcgen05.commit; owns the TMEM allocation
//   warps 5-12 producers  gather rows with 16-byte cp.async straight into the 128-byte-swizzled
//                         operand layout tcgen05 reads (no staging copy, no register round trip);
//                         eight warps because the load/store unit moves about 5 bytes per cycle per
//                         issuing warp for such gathers (measured: 20 B/cycle/SM with 4 warps, 40 with 8)
//   warp  13   index      streams the kernel-map entries of upcoming tiles (coalesced, bounds-checked)
//                         into a small shared-memory ring, several tiles ahead of everyone else, so
//                         that no other role ever waits on a dependent global load
//   warps 14-17 scatter   (forward / dgrad) read the patch back so that 8 or 16 consecutive lanes cover one
//                         destination row and issue vector red.global.add.  The SM's reduction path tops
//                         out near 25 bytes per cycle (measured); four warps that alternate between
//                         reading the patch and issuing reds get within about 20 % of it
//
// Shared-memory stages, index slots and the TMEM accumulator buffers are handed between the roles
// with mbarriers (one elected arrival per warp, one polling lane per warp).  Every wait is bounded
// (umma::mbar_wait): a wait that runs out makes all roles leave their loops, reports a problem and
// still frees the tensor memory.
//
// What these kernels replace in the reference: the wmma forward kernels (backend/fwd_kernels.cuh:17-144,
// backend/spconv.cuh:1328-1477, 1634-1776), the dgrad kernels (backend/bwd_kernels.cuh:13-142, 281-408)
// and the wgrad kernels (backend/bwd_kernels.cuh:419-527, 876-1368).  Differences that matter: a tile's
// gathered rows are loaded once and multiplied against the full output width (the reference re-gathers
// per 32 output columns, and wgrad per 32x32 weight tile), accumulation is fp32 for fp16 data, tiles
// come from the unpadded `kpos`, and every access is bounds-checked.
#pragma once

#include "common.cuh"
#include "umma.cuh"

namespace fgms {

constexpr int UMMA_THREADS = 448;       // wgrad: warps 0-13
constexpr int UMMA_GMS_THREADS = 576;   // forward / dgrad: four more warps for the scatter
constexpr int UMMA_SCATTER_WARPS = 4;
constexpr int UMMA_PROD_WARPS = 8;
constexpr int UMMA_PROD_THREADS = UMMA_PROD_WARPS * 32;
constexpr int UMMA_PROD_WARP0 = 5;
constexpr int UMMA_PROD_TID0 = UMMA_PROD_WARP0 * 32;
constexpr int UMMA_IDX_WARP = UMMA_PROD_WARP0 + UMMA_PROD_WARPS;   // 13
constexpr int UMMA_SCATTER_WARP0 = UMMA_IDX_WARP + 1;              // 14
constexpr int UMMA_EPI_WARPS = 4;
constexpr int UMMA_TILE_M = 128;      // pairs per forward / dgrad tile
constexpr int UMMA_STAGE_BYTES = 16384;
constexpr int UMMA_MAX_STAGES = 8;
constexpr int UMMA_IDX_SLOTS = 16;    // index-ring depth (tiles the index warp may run ahead)
constexpr int UMMA_IDX_BATCH = 4;     // tiles whose map entries the index warp loads at once
constexpr int UMMA_WG_MAX_PB = 64;    // pairs per wgrad stage, at most
constexpr int UMMA_PATCH_BYTES = UMMA_TILE_M * 256;  // one 256-byte block of every row of a tile
constexpr int UMMA_MAX_PATCHES = 2;  // patches are filled and scattered alternately when two fit

// shapes the tensor-core kernels take: both channel counts fill whole 128-byte spans, at most 256
inline bool umma_supported(int c_in, int c_out, int elem_bytes) {
  return (c_in * elem_bytes) % 128 == 0 && (c_out * elem_bytes) % 128 == 0 && c_in <= 256 && c_out <= 256;
}

// What the index warp publishes per tile.  Gather side (read by the producers; the MMA warp reads
// `seg` in wgrad) and scatter side (read by the epilogue) live in separate rings so that the slow
// consumer of one never holds back the other.
struct GatherSlot {
  int seg;     // segment (kernel offset, or k_vol for the dense centre term)
  int widx;    // weight matrix to use
  int cnt;     // valid pairs in the tile
  int pad;
  int g[UMMA_TILE_M];  // rows to gather (-1: skip).  wgrad: [0,64) input rows, [64,128) output rows
};
struct ScatterSlot {
  int s[UMMA_TILE_M];  // rows to accumulate into (-1: skip)
};

struct UmmaShared {
  uint64_t full[UMMA_MAX_STAGES];
  uint64_t empty[UMMA_MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t gidx_full[UMMA_IDX_SLOTS];
  uint64_t gidx_empty[UMMA_IDX_SLOTS];
  uint64_t sidx_full[UMMA_IDX_SLOTS];
  uint64_t sidx_empty[UMMA_IDX_SLOTS];
  uint64_t patch_full[2];
  uint64_t patch_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  GatherSlot gs[UMMA_IDX_SLOTS];
  ScatterSlot ss[UMMA_IDX_SLOTS];
};
constexpr int UMMA_SHARED_BYTES = (sizeof(UmmaShared) + 255) & ~255;
constexpr int UMMA_SMEM_FIXED = 1024 /* alignment slack */ + UMMA_SHARED_BYTES;

__device__ __forceinline__ uint8_t* align_1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}

__device__ __forceinline__ uint32_t tmem_cols_pow2(uint32_t need) {
  uint32_t c = 32;
  while (c < need) c <<= 1;
  return c;
}

// one lane polls, the warp learns the outcome
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = umma::mbar_wait(umma::smem_u32(bar), parity, abort_flag) ? 1 : 0;
  __syncwarp();  // orders the other lanes' later reads after what lane 0's acquire made visible
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// the warp has finished with something: one arrival for all 32 lanes
__device__ __forceinline__ void warp_arrive(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) umma::mbar_arrive(umma::smem_u32(bar));
}

__device__ __forceinline__ void init_barriers(UmmaShared* sh, int n_stage, int gidx_consumers, int sidx_consumers) {
  using namespace umma;
  for (int s = 0; s < n_stage; ++s) {
    mbar_init(smem_u32(&sh->full[s]), UMMA_PROD_THREADS);  // one hardware arrival per producer thread
    mbar_init(smem_u32(&sh->empty[s]), 1);
  }
  for (int b = 0; b < 2; ++b) {
    mbar_init(smem_u32(&sh->tmem_full[b]), 1);
    mbar_init(smem_u32(&sh->tmem_empty[b]), UMMA_EPI_WARPS);
    mbar_init(smem_u32(&sh->patch_full[b]), UMMA_EPI_WARPS);
    mbar_init(smem_u32(&sh->patch_empty[b]), UMMA_SCATTER_WARPS);
  }
  for (int i = 0; i < UMMA_IDX_SLOTS; ++i) {
    mbar_init(smem_u32(&sh->gidx_full[i]), 1);
    mbar_init(smem_u32(&sh->gidx_empty[i]), gidx_consumers);
    mbar_init(smem_u32(&sh->sidx_full[i]), 1);
    mbar_init(smem_u32(&sh->sidx_empty[i]), sidx_consumers > 0 ? sidx_consumers : 1);
  }
  sh->abort_flag = 0;
  mbar_fence_init();
}

// kpos copied to shared memory next to the tile table, so that tile bookkeeping never leaves the SM
__device__ __forceinline__ void load_kpos(const int32_t* __restrict__ kpos, int k_vol, int* kpos_s) {
  for (int s = threadIdx.x; s <= k_vol; s += blockDim.x) kpos_s[s] = __ldg(kpos + s);
}

// =============================================================================================
// forward / dgrad
//   A = gathered rows   [128 pairs x k_dim]  K-major, one 16 KB stage per 128-byte K chunk
//   B = W_k             forward: rows are the contraction index  -> MN-major operand
//                       dgrad  : rows are the output index (W^T)  -> K-major operand
//   D = [128 x n_dim] fp32 in TMEM, two buffers
// =============================================================================================
template <bool TF32, bool TRANS_W>
__global__ void __launch_bounds__(UMMA_GMS_THREADS, 1) umma_gms_kernel(GmsParams p, int n_stage, int n_patch) {
  using namespace umma;
  constexpr int ES = TF32 ? 4 : 2;
  constexpr int EPR = 128 / ES;  // elements per 128-byte span
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  const uint32_t w_bytes = (uint32_t)p.k_dim * p.n_dim * ES;
  uint8_t* sW = smem;
  uint8_t* sStage = smem + w_bytes;
  uint8_t* sEpi = sStage + (size_t)n_stage * UMMA_STAGE_BYTES;
  UmmaShared* sh = reinterpret_cast<UmmaShared*>(sEpi + (size_t)n_patch * UMMA_PATCH_BYTES);
  int* tile_start = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(sh) + UMMA_SHARED_BYTES);  // [k_vol + 2]
  int* kpos_s = tile_start + p.k_vol + 2;                                                         // [k_vol + 1]

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int n_seg = p.k_vol + 1;
  const int kch = p.k_dim / EPR;  // 128-byte K chunks per row
  volatile int* abort_flag = &sh->abort_flag;

  if (tid == 0) init_barriers(sh, n_stage, UMMA_PROD_WARPS, UMMA_SCATTER_WARPS);
  load_kpos(p.kpos, p.k_vol, kpos_s);
  build_tile_table(UMMA_TILE_M, p.kpos, p.k_vol, p.dense_rows, tile_start);  // syncs the CTA
  const uint32_t tmem_cols = tmem_cols_pow2(2u * p.n_dim);
  if (warp == 4) {
    tmem_alloc(smem_u32(&sh->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);
  bool ok = true;

  if (warp == UMMA_IDX_WARP) {
    // ------------------------------------------------------------------ index warp
    for (int tb = t0; tb < t1 && ok; tb += UMMA_IDX_BATCH) {
      const int nb = min(UMMA_IDX_BATCH, t1 - tb);
      int g[UMMA_IDX_BATCH][4], s[UMMA_IDX_BATCH][4], seg_[UMMA_IDX_BATCH], cnt_[UMMA_IDX_BATCH];
#pragma unroll
      for (int b = 0; b < UMMA_IDX_BATCH; ++b) {
        if (b < nb) {
          const int t = tb + b;
          const int seg = find_segment(tile_start, n_seg, t);
          const int lt = t - tile_start[seg];
          const bool dense = seg == p.k_vol;
          const int seg_base = dense ? 0 : kpos_s[seg];
          const int seg_cnt = dense ? p.dense_rows : (kpos_s[seg + 1] - seg_base);
          const int cnt = min(UMMA_TILE_M, seg_cnt - lt * UMMA_TILE_M);
          seg_[b] = seg;
          cnt_[b] = cnt;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int row = lane + 32 * q;
            const int j = lt * UMMA_TILE_M + row;
            int gv = -1, sv = -1;
            if (row < cnt) {
              gv = dense ? j : __ldg(p.gather_map + seg_base + j);
              sv = dense ? j : __ldg(p.scatter_map + seg_base + j);
            }
            g[b][q] = gv;
            s[b][q] = sv;
          }
        }
      }
#pragma unroll
      for (int b = 0; b < UMMA_IDX_BATCH; ++b) {
        if (b < nb && ok) {
          const int i = tb + b - t0;
          const int sl = i % UMMA_IDX_SLOTS;
          const uint32_t par = ((uint32_t)(i / UMMA_IDX_SLOTS) & 1u) ^ 1u;
          ok = warp_wait(&sh->gidx_empty[sl], par, abort_flag) && warp_wait(&sh->sidx_empty[sl], par, abort_flag);
          if (ok) {
            GatherSlot* gsl = &sh->gs[sl];
            ScatterSlot* ssl = &sh->ss[sl];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int row = lane + 32 * q;
              int gv = g[b][q], sv = s[b][q];
              if (row < cnt_[b] && (gv < 0 || gv >= p.n_gather || sv < 0 || sv >= p.n_scatter)) {
                report_problem();  // a map entry outside the tensors: the pair is skipped
                gv = sv = -1;
              }
              gsl->g[row] = gv;
              ssl->s[row] = sv;
            }
            if (lane == 0) {
              gsl->seg = seg_[b];
              gsl->widx = seg_[b] == p.k_vol ? p.dense_weight : seg_[b];
              gsl->cnt = cnt_[b];
            }
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(smem_u32(&sh->gidx_full[sl]));
              mbar_arrive(smem_u32(&sh->sidx_full[sl]));
            }
          }
        }
      }
    }
  } else if (warp >= UMMA_PROD_WARP0 && warp < UMMA_IDX_WARP) {
    // ------------------------------------------------------------------ producers
    const int tp = tid - UMMA_PROD_TID0;
    const int prow = tp >> 3, pc = tp & 7;  // thread gathers chunk pc of rows prow, prow + 32, prow + 64, prow + 96
    const uint32_t a_dst0 = (uint32_t)(prow >> 3) * 1024u + (uint32_t)(prow & 7) * 128u + (uint32_t)((pc ^ (prow & 7)) << 4);
    const uint8_t* src = static_cast<const uint8_t*>(p.src);
    const uint8_t* wts = static_cast<const uint8_t*>(p.weights);
    const size_t src_row_bytes = (size_t)p.k_dim * ES;
    const uint32_t w_row_bytes = (uint32_t)p.c_out * ES;
    int issued = 0, cur_w = -1;

    for (int t = t0; t < t1 && ok; ++t) {
      const int i = t - t0;
      const int sl = i % UMMA_IDX_SLOTS;
      ok = warp_wait(&sh->gidx_full[sl], (uint32_t)(i / UMMA_IDX_SLOTS) & 1u, abort_flag);
      if (!ok) break;
      const GatherSlot* slot = &sh->gs[sl];
      const int widx = slot->widx;
      int g[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) g[q] = slot->g[prow + 32 * q];
      warp_arrive(&sh->gidx_empty[sl]);

      const bool new_w = widx != cur_w;
      if (new_w) {
        // every MMA issued so far reads the old weights: wait until the last one has finished
        if (issued > 0) {
          const int last = issued - 1;
          ok = warp_wait(&sh->empty[last % n_stage], (uint32_t)(last / n_stage) & 1u, abort_flag);
          if (!ok) break;
        }
        cur_w = widx;
      }

      for (int kc = 0; kc < kch && ok; ++kc) {
        const int s = issued % n_stage;
        ok = warp_wait(&sh->empty[s], ((uint32_t)(issued / n_stage) & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        if (new_w && kc == 0) {
          const uint8_t* wk = wts + (size_t)widx * p.c_in * p.c_out * ES;
          const uint32_t sw = smem_u32(sW);
          if (!TRANS_W) {
            // rows = contraction index k (k_dim rows of n_dim elements): MN-major operand
            const int chunks_per_row = p.n_dim * ES / 16;
            const int total = p.k_dim * chunks_per_row;
            const uint32_t lbo = (uint32_t)p.k_dim * 128u;
            for (int e = tp; e < total; e += UMMA_PROD_THREADS) {
              const uint32_t row = e / chunks_per_row, c = e % chunks_per_row;
              const uint32_t off = TF32 ? mnmajor32_offset(row, c * 16u, lbo, 512u) : mnmajor_offset(row, c * 16u, lbo, 1024u);
              cp_async16(sw + off, wk + (size_t)row * w_row_bytes + c * 16u, true);
            }
          } else {
            // rows = output index n (n_dim rows of k_dim elements): K-major operand
            const int chunks_per_row = p.k_dim * ES / 16;
            const int total = p.n_dim * chunks_per_row;
            for (int e = tp; e < total; e += UMMA_PROD_THREADS) {
              const uint32_t row = e / chunks_per_row, c = e % chunks_per_row;
              cp_async16(sw + kmajor_offset(row, c * 16u, p.n_dim), wk + (size_t)row * w_row_bytes + c * 16u, true);
            }
          }
        }
        const uint32_t st = smem_u32(sStage + (size_t)s * UMMA_STAGE_BYTES) + a_dst0;
        const uint8_t* col = src + (size_t)kc * 128 + (size_t)pc * 16;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const bool valid = g[q] >= 0;
          cp_async16(st + (uint32_t)q * 4096u, valid ? col + (size_t)g[q] * src_row_bytes : src, valid);
        }
        // the stage's "full" barrier hears from this thread when everything it has issued has landed
        cp_async_arrive_noinc(smem_u32(&sh->full[s]));
        ++issued;
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc(TF32, false, !TRANS_W, UMMA_TILE_M, p.n_dim);
    const uint32_t sw = smem_u32(sW);
    int it = 0, tile_i = 0;
    for (int t = t0; t < t1 && ok; ++t, ++tile_i) {
      const int buf = tile_i & 1;
      ok = warp_wait(&sh->tmem_empty[buf], ((uint32_t)(tile_i >> 1) & 1u) ^ 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)buf * p.n_dim;
      for (int kc = 0; kc < kch && ok; ++kc, ++it) {
        const int s = it % n_stage;
        ok = warp_wait(&sh->full[s], (uint32_t)(it / n_stage) & 1u, abort_flag);
        if (!ok) break;
        if (lane == 0) {
          fence_proxy_async();  // the stage was written through cp.async; the MMA reads it through the async proxy
          tc_fence_after();
          const uint32_t sa = smem_u32(sStage + (size_t)s * UMMA_STAGE_BYTES);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t a_desc = make_sdesc(sa + ks * 32u, 16u, 1024u);
            uint64_t b_desc;
            if (!TRANS_W) {
              // MN-major B: step (kc*EPR + ks*UMMA_K) rows of 128 bytes into the weight tile
              const uint32_t k_row = (uint32_t)kc * EPR + (uint32_t)ks * (32u / ES);
              b_desc = make_sdesc(sw + k_row * 128u, (uint32_t)p.k_dim * 128u, TF32 ? 512u : 1024u, TF32 ? 1u : 2u);
            } else {
              b_desc = make_sdesc(sw + (uint32_t)kc * ((uint32_t)p.n_dim * 128u) + ks * 32u, 16u, 1024u);
            }
            mma_ss<TF32>(d_tmem, a_desc, b_desc, idesc, (kc | ks) != 0);
          }
          mma_commit(smem_u32(&sh->empty[s]));
          if (kc == kch - 1) mma_commit(smem_u32(&sh->tmem_full[buf]));
        }
        __syncwarp();
      }
    }
  } else if (warp >= UMMA_SCATTER_WARP0) {
    // ------------------------------------------------------------------ scatter (warps 14-17)
    // Warp w owns tile rows [32 w, 32 w + 32).  It reads a parked 256-byte block back so that `cpr`
    // consecutive lanes cover one row, and adds it to the destination row with 16-byte vector reds.
    const int sw_i = warp - UMMA_SCATTER_WARP0;
    uint8_t* dst = static_cast<uint8_t*>(p.dst);
    const uint32_t row_bytes = (uint32_t)p.n_dim * ES;
    uint32_t blk_i = 0;
    int tile_i = 0;
    for (int t = t0; t < t1 && ok; ++t, ++tile_i) {
      const int sl = tile_i % UMMA_IDX_SLOTS;
      ok = warp_wait(&sh->sidx_full[sl], (uint32_t)(tile_i / UMMA_IDX_SLOTS) & 1u, abort_flag);
      if (!ok) break;
      const int srow = sh->ss[sl].s[sw_i * 32 + lane];
      warp_arrive(&sh->sidx_empty[sl]);
      for (uint32_t cb = 0; cb < row_bytes && ok; cb += 256, ++blk_i) {
        const uint32_t pb = blk_i % (uint32_t)n_patch;
        ok = warp_wait(&sh->patch_full[pb], (blk_i / (uint32_t)n_patch) & 1u, abort_flag);
        if (!ok) break;
        const uint32_t blk_bytes = min(256u, row_bytes - cb);
        const uint32_t cpr = blk_bytes >> 4;  // 16-byte chunks per row in this block: 8 or 16
        const uint32_t rpi = 32 / cpr;        // rows one warp-wide instruction covers: 4 or 2
        const uint32_t ch = lane % cpr, rsub = lane / cpr;
        const uint8_t* patch = sEpi + pb * UMMA_PATCH_BYTES + (size_t)(sw_i * 32) * 256;
        uint8_t* dcol = dst + cb + (ch << 4);
#pragma unroll 1
        for (uint32_t r0 = 0; r0 < 32; r0 += 8 * rpi) {  // cpr = 16: two rounds of 8 reds; cpr = 8: one
          uint4 v[8];
          int sr[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t r = r0 + u * rpi + rsub;  // row within this warp's 32
            v[u] = *reinterpret_cast<const uint4*>(patch + r * 256 + ((ch ^ (r & 7)) << 4));
            sr[u] = __shfl_sync(0xffffffffu, srow, r);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (sr[u] >= 0) {
              uint8_t* o = dcol + (size_t)sr[u] * row_bytes;
              if (TF32) red_add_v4(reinterpret_cast<float*>(o), __uint_as_float(v[u].x), __uint_as_float(v[u].y),
                                   __uint_as_float(v[u].z), __uint_as_float(v[u].w));
              else red_add_h8(reinterpret_cast<__half*>(o), v[u].x, v[u].y, v[u].z, v[u].w);
            }
          }
        }
        warp_arrive(&sh->patch_empty[pb]);  // every lane has its data in registers and has issued its reds
      }
    }
  } else {
    // ------------------------------------------------------------------ drain (warps 0-3)
    // Each thread owns one accumulator row (its TMEM lane): it converts the row block by block
    // (256 bytes of output at a time) and parks it, 16-byte chunks XOR-swizzled by row, in the patch.
    const uint32_t row_bytes = (uint32_t)p.n_dim * ES;
    int tile_i = 0;
    uint32_t blk_i = 0;
    for (int t = t0; t < t1 && ok; ++t, ++tile_i) {
      const int buf = tile_i & 1;
      ok = warp_wait(&sh->tmem_full[buf], (uint32_t)(tile_i >> 1) & 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)buf * p.n_dim;
      for (uint32_t cb = 0; cb < row_bytes && ok; cb += 256, ++blk_i) {
        const uint32_t blk_bytes = min(256u, row_bytes - cb);
        const uint32_t ncol = blk_bytes / ES;
        const uint32_t col0 = cb / ES;
        const uint32_t pb = blk_i % (uint32_t)n_patch;
        ok = warp_wait(&sh->patch_empty[pb], ((blk_i / (uint32_t)n_patch) & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        uint8_t* mine = sEpi + pb * UMMA_PATCH_BYTES + (size_t)tid * 256;
        const uint32_t sw7 = (uint32_t)(tid & 7);
        for (uint32_t c0 = 0; c0 < ncol; c0 += 32) {
          uint32_t v0[16], v1[16];
          tmem_ld16(taddr + col0 + c0, v0);
          tmem_ld16(taddr + col0 + c0 + 16, v1);
          tmem_ld_wait();
          if (TF32) {
            const uint32_t ch0 = c0 / 4;  // first 16-byte chunk of these 32 columns
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              *reinterpret_cast<uint4*>(mine + (((ch0 + q) ^ sw7) << 4)) = make_uint4(v0[4 * q], v0[4 * q + 1], v0[4 * q + 2], v0[4 * q + 3]);
              *reinterpret_cast<uint4*>(mine + (((ch0 + 4 + q) ^ sw7) << 4)) = make_uint4(v1[4 * q], v1[4 * q + 1], v1[4 * q + 2], v1[4 * q + 3]);
            }
          } else {
            const uint32_t ch0 = c0 / 8;
            uint32_t h[16];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              h[q] = pack_half2(__uint_as_float(v0[2 * q]), __uint_as_float(v0[2 * q + 1]));
              h[8 + q] = pack_half2(__uint_as_float(v1[2 * q]), __uint_as_float(v1[2 * q + 1]));
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<uint4*>(mine + (((ch0 + q) ^ sw7) << 4)) = make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
          }
        }
        if (cb + 256 >= row_bytes) {
          // accumulator fully read: hand the TMEM buffer back
          tc_fence_before();
          warp_arrive(&sh->tmem_empty[buf]);
        }
        warp_arrive(&sh->patch_full[pb]);
      }
    }
  }

  if (!ok && lane == 0) report_problem();
  cp_async_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, tmem_cols);
}

// =============================================================================================
// wgrad:  dw[k] (c_in x c_out, fp32) += sum over the pairs of offset k of feats[in]^T (x) out_grad[out]
//   the pair index is the contraction index: both operands are gathered rows used MN-major
//   A = feats rows     [pb pairs x c_in ]   M = c_in  (tiles of 128 rows, or one tile of 64)
//   B = out_grad rows  [pb pairs x c_out]   N = c_out
//   The accumulator stays in TMEM while the CTA walks consecutive stages of the same offset and is
//   flushed with vector red.global.add.f32 when the offset changes (split-K across CTAs).
// =============================================================================================
struct WgradTiling {
  int pb;          // pairs per stage (multiple of 16, at most UMMA_WG_MAX_PB)
  int n_mtile;     // 1 or 2 accumulator row tiles
  int mtile_m;     // rows of each tile's MMA: 128 or 64
  int alias;       // 1: the single tile has fewer real rows than mtile_m; extra rows repeat (LBO = 0)
  int n_buf;       // TMEM accumulator sets (2 when they fit)
  int n_stage;
};

template <bool TF32>
__global__ void __launch_bounds__(UMMA_THREADS, 1) umma_wgrad_kernel(WgradParams p, WgradTiling tl) {
  using namespace umma;
  constexpr int ES = TF32 ? 4 : 2;
  constexpr int UK = 32 / ES;  // contraction length of one MMA
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  const uint32_t a_bytes = (uint32_t)tl.pb * p.c_in * ES;
  const uint32_t stage_bytes = (uint32_t)tl.pb * (p.c_in + p.c_out) * ES;
  uint8_t* sStage = smem;
  UmmaShared* sh = reinterpret_cast<UmmaShared*>(sStage + (size_t)tl.n_stage * stage_bytes);
  int* tile_start = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(sh) + UMMA_SHARED_BYTES);
  int* kpos_s = tile_start + p.k_vol + 2;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int n_seg = p.k_vol + 1;
  const int n_stage = tl.n_stage;
  volatile int* abort_flag = &sh->abort_flag;
  const uint32_t lbo = (uint32_t)tl.pb * 128u;  // next 128 bytes of every gathered row
  const uint32_t buf_cols = (uint32_t)tl.n_mtile * p.c_out;

  if (tid == 0) init_barriers(sh, n_stage, UMMA_PROD_WARPS + 1, 0);
  load_kpos(p.kpos, p.k_vol, kpos_s);
  build_tile_table(tl.pb, p.kpos, p.k_vol, 0, tile_start);
  const uint32_t tmem_cols = tmem_cols_pow2(buf_cols * tl.n_buf);
  if (warp == 4) {
    tmem_alloc(smem_u32(&sh->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);
  bool ok = true;

  if (warp == UMMA_IDX_WARP) {
    // ------------------------------------------------------------------ index warp (pb <= 64 pairs per stage)
    for (int tb = t0; tb < t1 && ok; tb += UMMA_IDX_BATCH) {
      const int nb = min(UMMA_IDX_BATCH, t1 - tb);
      int iv[UMMA_IDX_BATCH][2], ov[UMMA_IDX_BATCH][2], seg_[UMMA_IDX_BATCH], cnt_[UMMA_IDX_BATCH];
#pragma unroll
      for (int b = 0; b < UMMA_IDX_BATCH; ++b) {
        if (b < nb) {
          const int t = tb + b;
          const int seg = find_segment(tile_start, n_seg, t);
          const int lt = t - tile_start[seg];
          const int seg_base = kpos_s[seg];
          const int cnt = min(tl.pb, kpos_s[seg + 1] - seg_base - lt * tl.pb);
          seg_[b] = seg;
          cnt_[b] = cnt;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int row = lane + 32 * q;
            int a = -1, o = -1;
            if (row < cnt) {
              a = __ldg(p.in_map + seg_base + lt * tl.pb + row);
              o = __ldg(p.out_map + seg_base + lt * tl.pb + row);
            }
            iv[b][q] = a;
            ov[b][q] = o;
          }
        }
      }
#pragma unroll
      for (int b = 0; b < UMMA_IDX_BATCH; ++b) {
        if (b < nb && ok) {
          const int i = tb + b - t0;
          const int sl = i % UMMA_IDX_SLOTS;
          ok = warp_wait(&sh->gidx_empty[sl], ((uint32_t)(i / UMMA_IDX_SLOTS) & 1u) ^ 1u, abort_flag);
          if (ok) {
            GatherSlot* slot = &sh->gs[sl];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int row = lane + 32 * q;
              int a = iv[b][q], o = ov[b][q];
              if (row < cnt_[b] && (a < 0 || a >= p.n_in || o < 0 || o >= p.n_out)) {
                report_problem();
                a = o = -1;
              }
              slot->g[row] = a;
              slot->g[UMMA_WG_MAX_PB + row] = o;
            }
            if (lane == 0) {
              slot->seg = seg_[b];
              slot->cnt = cnt_[b];
            }
            warp_arrive(&sh->gidx_full[sl]);
          }
        }
      }
    }
  } else if (warp >= UMMA_PROD_WARP0 && warp < UMMA_IDX_WARP) {
    // ------------------------------------------------------------------ producers
    const int tp = tid - UMMA_PROD_TID0;
    const uint8_t* feats = static_cast<const uint8_t*>(p.feats);
    const uint8_t* og = static_cast<const uint8_t*>(p.out_grad);
    const int ca = p.c_in * ES / 16, cb = p.c_out * ES / 16;  // 16-byte chunks per row
    const int total_a = tl.pb * ca, total_b = tl.pb * cb;
    const size_t a_row_bytes = (size_t)p.c_in * ES, b_row_bytes = (size_t)p.c_out * ES;
    // Thread tp owns the 16-byte chunks e = tp, tp + 256, ... (at most 4 per operand) of every stage:
    // chunk e is (row e / cpr, column chunk e % cpr).  Row, source column offset and shared-memory
    // offset of each owned chunk are fixed for the whole kernel, so the stage loop has no address
    // arithmetic beyond one multiply-add per chunk.
    int a_row[4], b_row[4];
    uint32_t a_dst[4], b_dst[4], a_col[4], b_col[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = tp + u * UMMA_PROD_THREADS;
      a_row[u] = e < total_a ? e / ca : -1;
      b_row[u] = e < total_b ? e / cb : -1;
      const uint32_t ac = e < total_a ? (uint32_t)(e % ca) : 0u, bc = e < total_b ? (uint32_t)(e % cb) : 0u;
      a_col[u] = ac * 16u;
      b_col[u] = bc * 16u;
      const uint32_t ar = a_row[u] < 0 ? 0u : (uint32_t)a_row[u], br = b_row[u] < 0 ? 0u : (uint32_t)b_row[u];
      a_dst[u] = TF32 ? mnmajor32_offset(ar, ac * 16u, lbo, 512u) : mnmajor_offset(ar, ac * 16u, lbo, 1024u);
      b_dst[u] = a_bytes + (TF32 ? mnmajor32_offset(br, bc * 16u, lbo, 512u) : mnmajor_offset(br, bc * 16u, lbo, 1024u));
    }

    int issued = 0;
    for (int t = t0; t < t1 && ok; ++t) {
      const int i = t - t0;
      const int sl = i % UMMA_IDX_SLOTS;
      ok = warp_wait(&sh->gidx_full[sl], (uint32_t)(i / UMMA_IDX_SLOTS) & 1u, abort_flag);
      if (!ok) break;
      const GatherSlot* slot = &sh->gs[sl];
      const int s = issued % n_stage;
      ok = warp_wait(&sh->empty[s], ((uint32_t)(issued / n_stage) & 1u) ^ 1u, abort_flag);
      if (!ok) break;
      const uint32_t sa = smem_u32(sStage + (size_t)s * stage_bytes);
      int ia[4], ib[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        ia[u] = a_row[u] >= 0 ? slot->g[a_row[u]] : -1;
        ib[u] = b_row[u] >= 0 ? slot->g[UMMA_WG_MAX_PB + b_row[u]] : -1;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (a_row[u] >= 0) {
          const bool valid = ia[u] >= 0;
          cp_async16(sa + a_dst[u], valid ? feats + ((size_t)ia[u] * a_row_bytes + a_col[u]) : feats, valid);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (b_row[u] >= 0) {
          const bool valid = ib[u] >= 0;
          cp_async16(sa + b_dst[u], valid ? og + ((size_t)ib[u] * b_row_bytes + b_col[u]) : og, valid);
        }
      }
      cp_async_arrive_noinc(smem_u32(&sh->full[s]));
      warp_arrive(&sh->gidx_empty[sl]);
      ++issued;
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc(TF32, true, true, tl.mtile_m, p.c_out);
    const uint32_t sbo = TF32 ? 512u : 1024u, ltype = TF32 ? 1u : 2u;
    const uint32_t a_lbo = tl.alias ? 0u : lbo;
    const uint32_t mtile_stride = (uint32_t)(tl.mtile_m * ES / 128) * lbo;  // A start of the second row tile
    int it = 0, run_i = 0, cur_seg = -1;
    bool first = true;
    for (int t = t0; t < t1 && ok; ++t, ++it) {
      const int sl = it % UMMA_IDX_SLOTS;
      ok = warp_wait(&sh->gidx_full[sl], (uint32_t)(it / UMMA_IDX_SLOTS) & 1u, abort_flag);
      if (!ok) break;
      const int seg = sh->gs[sl].seg;
      warp_arrive(&sh->gidx_empty[sl]);
      if (seg != cur_seg) {
        if (cur_seg >= 0) {
          if (lane == 0) mma_commit(smem_u32(&sh->tmem_full[(run_i % tl.n_buf)]));
          __syncwarp();
          ++run_i;
        }
        cur_seg = seg;
        first = true;
        const int buf = run_i % tl.n_buf;
        const int use = run_i / tl.n_buf;
        ok = warp_wait(&sh->tmem_empty[buf], ((uint32_t)use & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
      }
      const int buf = run_i % tl.n_buf;
      const int s = it % n_stage;
      ok = warp_wait(&sh->full[s], (uint32_t)(it / n_stage) & 1u, abort_flag);
      if (!ok) break;
      if (lane == 0) {
        fence_proxy_async();
        tc_fence_after();
        const uint32_t sa = smem_u32(sStage + (size_t)s * stage_bytes);
        const uint32_t sb = sa + a_bytes;
        for (int ks = 0; ks < tl.pb / UK; ++ks) {
          const uint32_t kadv = (uint32_t)ks * UK * 128u;
          const uint64_t b_desc = make_sdesc(sb + kadv, lbo, sbo, ltype);
          for (int mt = 0; mt < tl.n_mtile; ++mt) {
            const uint64_t a_desc = make_sdesc(sa + kadv + mt * mtile_stride, a_lbo, sbo, ltype);
            mma_ss<TF32>(tmem_base + (uint32_t)buf * buf_cols + (uint32_t)mt * p.c_out, a_desc, b_desc, idesc,
                         !(first && ks == 0));
          }
        }
        mma_commit(smem_u32(&sh->empty[s]));
      }
      __syncwarp();
      first = false;
    }
    if (ok && cur_seg >= 0) {
      if (lane == 0) mma_commit(smem_u32(&sh->tmem_full[(run_i % tl.n_buf)]));
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3)
    int run_i = 0;
    int t = t0;
    while (t < t1 && ok) {
      const int seg = find_segment(tile_start, n_seg, t);
      const int seg_end = min(t1, tile_start[seg + 1]);  // this CTA's stages of the offset end here
      t = seg_end;
      const int buf = run_i % tl.n_buf;
      const int use = run_i / tl.n_buf;
      ok = warp_wait(&sh->tmem_full[buf], (uint32_t)use & 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      float* dwk = p.dw + (size_t)seg * p.c_in * p.c_out;
      for (int mt = 0; mt < tl.n_mtile; ++mt) {
        // accumulator row held by this thread's TMEM lane
        int m;
        if (tl.mtile_m == 128) m = mt * 128 + tid;
        else m = (lane < 16) ? (warp * 16 + lane) : -1;  // M = 64: row i lives in lane (i/16)*32 + i%16
        const bool valid = m >= 0 && m < p.c_in;
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)buf * buf_cols + (uint32_t)mt * p.c_out;
        float* orow = dwk + (size_t)(valid ? m : 0) * p.c_out;
        for (int c0 = 0; c0 < p.c_out; c0 += 32) {
          uint32_t v0[16], v1[16];
          tmem_ld16(taddr + c0, v0);
          tmem_ld16(taddr + c0 + 16, v1);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              red_add_v4(orow + c0 + 4 * q, __uint_as_float(v0[4 * q]), __uint_as_float(v0[4 * q + 1]),
                         __uint_as_float(v0[4 * q + 2]), __uint_as_float(v0[4 * q + 3]));
#pragma unroll
            for (int q = 0; q < 4; ++q)
              red_add_v4(orow + c0 + 16 + 4 * q, __uint_as_float(v1[4 * q]), __uint_as_float(v1[4 * q + 1]),
                         __uint_as_float(v1[4 * q + 2]), __uint_as_float(v1[4 * q + 3]));
          }
        }
      }
      tc_fence_before();
      warp_arrive(&sh->tmem_empty[buf]);
      ++run_i;
    }
  }

  if (!ok && lane == 0) report_problem();
  cp_async_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, tmem_cols);
}

// =============================================================================================
// host launchers: return 0 after a launch, 1 when the shape or the pointers do not fit the
// tensor-core kernel (the caller then takes the CUDA-core path), < 0 on a CUDA error.
// =============================================================================================
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int umma_table_bytes(int k_vol) { return ((2 * k_vol + 3) * 4 + 15) & ~15; }

// cudaFuncSetAttribute is needed once per device and kernel; remember what was granted
template <typename K>
inline int ensure_smem(K kernel, int bytes, int slot) {
  static int granted[8][64] = {};  // [kernel slot][device]
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (dev < 0 || dev >= 64) return -1;
  if (granted[slot][dev] >= bytes) return 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -1;
  granted[slot][dev] = bytes;
  return 0;
}

inline int launch_umma_gms(const GmsParams& p, bool trans, bool f16, cudaStream_t st, int sms, int max_smem) {
  const int es = f16 ? 2 : 4;
  if (!aligned16(p.src) || !aligned16(p.weights) || !aligned16(p.dst)) return 1;
  const int w_bytes = p.k_dim * p.n_dim * es;
  const int fixed = UMMA_SMEM_FIXED + umma_table_bytes(p.k_vol);
  int n_patch = UMMA_MAX_PATCHES;
  int n_stage = (max_smem - fixed - w_bytes - n_patch * UMMA_PATCH_BYTES) / UMMA_STAGE_BYTES;
  if (n_stage < 4) {  // large weight tiles: give the second patch's room to the gather stages
    n_patch = 1;
    n_stage = (max_smem - fixed - w_bytes - n_patch * UMMA_PATCH_BYTES) / UMMA_STAGE_BYTES;
  }
  if (n_stage > UMMA_MAX_STAGES) n_stage = UMMA_MAX_STAGES;
  if (n_stage < 2) return 1;
  const int smem = fixed + w_bytes + n_patch * UMMA_PATCH_BYTES + n_stage * UMMA_STAGE_BYTES;
  int rc;
  if (f16) {
    if (trans) { rc = ensure_smem(umma_gms_kernel<false, true>, max_smem, 0); if (rc) return rc; umma_gms_kernel<false, true><<<sms, UMMA_GMS_THREADS, smem, st>>>(p, n_stage, n_patch); }
    else       { rc = ensure_smem(umma_gms_kernel<false, false>, max_smem, 1); if (rc) return rc; umma_gms_kernel<false, false><<<sms, UMMA_GMS_THREADS, smem, st>>>(p, n_stage, n_patch); }
  } else {
    if (trans) { rc = ensure_smem(umma_gms_kernel<true, true>, max_smem, 2); if (rc) return rc; umma_gms_kernel<true, true><<<sms, UMMA_GMS_THREADS, smem, st>>>(p, n_stage, n_patch); }
    else       { rc = ensure_smem(umma_gms_kernel<true, false>, max_smem, 3); if (rc) return rc; umma_gms_kernel<true, false><<<sms, UMMA_GMS_THREADS, smem, st>>>(p, n_stage, n_patch); }
  }
  return 0;
}

// Accumulator row tiling for c_in: whole 128-row tiles, or a single 64-row tile, or a single tile whose
// rows beyond c_in repeat the real ones.  Returns false for row counts not covered (e.g. 192).
inline bool wgrad_tiling(int c_in, int c_out, int es, int max_smem, int k_vol, WgradTiling* tl) {
  const int span = 128 / es;  // rows per 128-byte span of a gathered feature row
  if (c_in % 128 == 0) { tl->n_mtile = c_in / 128; tl->mtile_m = 128; tl->alias = 0; }
  else if (c_in == 64) { tl->n_mtile = 1; tl->mtile_m = 64; tl->alias = 0; }
  else if (c_in == span) { tl->n_mtile = 1; tl->mtile_m = 64; tl->alias = 1; }  // tf32, 32 rows
  else return false;
  if (tl->n_mtile > 2) return false;
  if (tl->n_mtile * c_out > 512) return false;
  tl->n_buf = (2 * tl->n_mtile * c_out <= 512) ? 2 : 1;
  const int row_bytes = (c_in + c_out) * es;
  int pb = UMMA_STAGE_BYTES / row_bytes;
  pb = pb / 16 * 16;
  if (pb < 16) pb = 16;
  if (pb > UMMA_WG_MAX_PB) pb = UMMA_WG_MAX_PB;
  tl->pb = pb;
  int n_stage = (max_smem - UMMA_SMEM_FIXED - umma_table_bytes(k_vol)) / (pb * row_bytes);
  if (n_stage > UMMA_MAX_STAGES) n_stage = UMMA_MAX_STAGES;
  if (n_stage < 2) return false;
  tl->n_stage = n_stage;
  return true;
}

inline int launch_umma_wgrad(const WgradParams& p, bool f16, cudaStream_t st, int sms, int max_smem) {
  const int es = f16 ? 2 : 4;
  if (!aligned16(p.feats) || !aligned16(p.out_grad) || !aligned16(p.dw)) return 1;
  WgradTiling tl;
  if (!wgrad_tiling(p.c_in, p.c_out, es, max_smem, p.k_vol, &tl)) return 1;
  const int smem = UMMA_SMEM_FIXED + umma_table_bytes(p.k_vol) + tl.n_stage * tl.pb * (p.c_in + p.c_out) * es;
  int rc;
  if (f16) { rc = ensure_smem(umma_wgrad_kernel<false>, max_smem, 4); if (rc) return rc; umma_wgrad_kernel<false><<<sms, UMMA_THREADS, smem, st>>>(p, tl); }
  else     { rc = ensure_smem(umma_wgrad_kernel<true>, max_smem, 5); if (rc) return rc; umma_wgrad_kernel<true><<<sms, UMMA_THREADS, smem, st>>>(p, tl); }
  return 0;
}

}  // namespace fgms
