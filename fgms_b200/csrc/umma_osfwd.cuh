// Output-stationary forward on tcgen05: every output row is produced by ONE accumulator and written once.
//
//   out[r] (=, +=) act( sum_k in[nbr[k][r]] * W[k]  (+ bias) )        for the output rows r of a tile
//
// The scatter form (umma_gms3.cuh, the reference's scheme, backend/fwd_kernels.cuh:130-141) walks the pair list
// offset by offset and adds every pair's product to its output row with an atomic, so an output row receives up
// to k_vol atomics in an order that changes from run to run, and nothing can be applied to the finished row
// inside the kernel.  Here the map is a neighbour table nbr[k][r] (input row of output row r under offset k, -1
// for none; built from the pair list by os_fill_nbr_kernel): a tile is 128 consecutive output rows, its
// accumulator stays in tensor memory while the CTA walks all k_vol offsets (rows without a neighbour are
// zero-filled), and the epilogue adds the bias, applies ReLU and stores the rows — plain stores, the same bits on
// every run.  Up to four tiles (as many accumulators as the 512 TMEM columns hold) are walked together, offset
// by offset, so that a weight matrix is staged once per group of tiles and offset.
//
// The price is one 128-row stage per (tile, offset) however few of the tile's rows have a neighbour there:
// k_vol stages per 128 output rows against pairs / 128 stages in the scatter form — measured 0.9-1.1 times the
// scatter form's time on fully occupied grids, 2.6 times at 9.5 pairs per voxel, 8 times at 2.1.  It is the form
// for callers to whom reproducible bits or the fused epilogue are worth the extra stages.
//
// Roles (13 warps): 8 producers (16-byte cp.async gathers into the K-major 128-byte-swizzled stage ring, weight
// matrices into one of two buffers), one MMA warp, 4 epilogue warps.  All waits are bounded.
#pragma once
#include "common.cuh"
#include "umma.cuh"
#include "umma_gms3.cuh"  // G3Config / g3_plan (operand and stage sizes), g3_wait, G3_STAGE_BYTES

namespace fgms {

constexpr int OS_EPI_WARPS = 4;
constexpr int OS_MMA_WARP = 4;
constexpr int OS_PROD_WARP0 = 5;
constexpr int OS_PROD_WARPS = 8;
constexpr int OS_PROD_THREADS = OS_PROD_WARPS * 32;
constexpr int OS_THREADS = (OS_PROD_WARP0 + OS_PROD_WARPS) * 32;  // 416
constexpr int OS_PREFETCH = 4;  // neighbour entries are fetched this many stages ahead
constexpr int OS_TILE = 128;

struct OsParams {
  const void* src;       // [n_in , c_in ]
  const void* weights;   // [k_vol, c_in, c_out]
  void* dst;             // [n_out, c_out]
  const int32_t* nbr;    // [k_vol][nbr_stride]: input row of output row r under offset k, -1 for none
  const void* bias;      // [c_out] in the storage type, or null
  long long nbr_stride;  // entries per offset: n_tiles * 128
  int n_in, n_out, n_tiles;
  int c_in, c_out, k_vol;
  int relu;        // 1: max(x, 0) after the bias
  int accumulate;  // 1: out += result (what the reference's forward does); 0: out = result
};

struct OsShared {
  uint64_t full[G3_MAX_STAGES];
  uint64_t empty[G3_MAX_STAGES];
  uint64_t tmem_full[4];
  uint64_t tmem_empty[4];
  uint64_t w_free[2];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int OS_SHARED_BYTES = (sizeof(OsShared) + 15) & ~15;

// The walk every role makes over the CTA's tiles [.., t1): groups of up to `gsz` consecutive tiles; within a group
// offset by offset, within an offset tile by tile.  A CTA's tile range is cut to the tile (not to the group), so the
// CTAs' loads differ by one tile at most; the last group of a CTA may be smaller.
struct OsWalk {
  int tb, k, g, gv;  // first tile of the group, offset, tile of the group, tiles this group has (<= 0: past the end)
  __device__ __forceinline__ void init(int t0, int gsz, int t1) {
    tb = t0; k = 0; g = 0;
    gv = min(gsz, t1 - tb);
  }
  __device__ __forceinline__ void next(int gsz, int t1, int k_vol) {
    if (++g >= gv) {
      g = 0;
      if (++k == k_vol) {
        k = 0;
        tb += gsz;
        gv = min(gsz, t1 - tb);
      }
    }
  }
  __device__ __forceinline__ int tile() const { return tb + g; }
};

// nbr[k][out_map[j]] = in_map[j] for every pair j of offset k (the table is filled with -1 beforehand).  Every kpos
// entry is clamped to [0, map_len]; a pair with an entry outside the tensors is skipped and counted.
__global__ void os_fill_nbr_kernel(const int32_t* __restrict__ kpos, const int32_t* __restrict__ in_map,
                                   const int32_t* __restrict__ out_map, long long map_len, int n_in, int n_out, int k_vol,
                                   long long stride, int32_t* __restrict__ nbr) {
  extern __shared__ int kp[];  // [k_vol + 1], clamped
  for (int i = threadIdx.x; i <= k_vol; i += blockDim.x) {
    long long v = kpos[i];
    kp[i] = (int)(v < 0 ? 0 : (v > map_len ? map_len : v));
  }
  __syncthreads();
  const long long total = kp[k_vol];
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += (long long)gridDim.x * blockDim.x) {
    int lo = 0, hi = k_vol;  // the offset k with kp[k] <= j < kp[k + 1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (kp[mid] <= j) lo = mid; else hi = mid;
    }
    const int i = in_map[j], o = out_map[j];
    if ((unsigned)i < (unsigned)n_in && (unsigned)o < (unsigned)n_out) nbr[(long long)lo * stride + o] = i;
    else report_problem();
  }
}

template <bool TF32>
__global__ void __launch_bounds__(OS_THREADS, 1) umma_osfwd_kernel(OsParams p, G3Config cfg) {
  using namespace umma;
  constexpr int ES = TF32 ? 4 : 2;
  constexpr int EPR = 128 / ES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sW = smem;
  uint8_t* sStage = sW + (size_t)cfg.n_wbuf * cfg.w_bytes;
  uint8_t* sPatch = sStage + (size_t)cfg.n_stage * G3_STAGE_BYTES;
  OsShared* sh = reinterpret_cast<OsShared*>(sPatch + G3_PATCH_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kch = cfg.kch, n_stage = cfg.n_stage, gsz = cfg.n_tbuf;
  const int k_bytes = p.c_in * ES;
  volatile int* abort_flag = &sh->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < n_stage; ++s) {
      mbar_init(smem_u32(&sh->full[s]), OS_PROD_THREADS);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(smem_u32(&sh->tmem_full[b]), 1);
      mbar_init(smem_u32(&sh->tmem_empty[b]), OS_EPI_WARPS);
    }
    mbar_init(smem_u32(&sh->w_free[0]), 1);
    mbar_init(smem_u32(&sh->w_free[1]), 1);
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)(gsz * cfg.n_acc)) tmem_cols <<= 1;
  if (warp == OS_MMA_WARP) {
    tmem_alloc(smem_u32(&sh->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  griddep_wait();
  griddep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  // this CTA's tiles
  int t0, t1;
  cta_tile_range(p.n_tiles, &t0, &t1);
  bool ok = true;

  if (t0 >= t1) {
    // nothing for this CTA
  } else if (warp >= OS_PROD_WARP0) {
    // ------------------------------------------------------------------ producers
    // Warp pw owns tile rows [16 pw, 16 pw + 16); lane (rs, pc) = (lane / 8, lane % 8) copies 16-byte chunk pc of
    // every 128-byte K chunk of the rows rs, rs + 4, rs + 8, rs + 12 of that block.
    const int pw = warp - OS_PROD_WARP0;
    const int tp = tid - OS_PROD_WARP0 * 32;
    const int rs = lane >> 3, pc = lane & 7;
    const uint8_t* src = static_cast<const uint8_t*>(p.src);
    const uint8_t* wts = static_cast<const uint8_t*>(p.weights);
    uint32_t a_dst[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t r = (uint32_t)(16 * pw + rs + 4 * j);
      a_dst[j] = (r >> 3) * 1024u + (r & 7u) * 128u + (((uint32_t)pc ^ (r & 7u)) << 4);
    }
    // lane r < 16 fetches the neighbour entry of the warp's row r
    auto load_entry = [&](const OsWalk& w) -> int {
      if (lane >= 16) return -1;
      return __ldg(p.nbr + (long long)w.k * p.nbr_stride + (long long)w.tile() * OS_TILE + 16 * pw + lane);
    };
    // weight matrix W_k -> MN-major operand (rows = contraction index), as in the scatter-form forward
    const int cpr = p.c_out * ES / 16;  // 16-byte chunks per row of W_k
    const uint32_t w_row_bytes = (uint32_t)p.c_out * ES;
    const uint32_t w_lbo = (uint32_t)p.c_in * 128u;
    auto load_weights = [&](int k, int wb) {
      const uint8_t* wk = wts + (size_t)k * p.c_in * p.c_out * ES;
      const uint32_t sw = smem_u32(sW + (size_t)wb * cfg.w_bytes);
      const int total = p.c_in * cpr;
      for (int e = tp; e < total; e += OS_PROD_THREADS) {
        const uint32_t row = e / cpr, c = e % cpr;
        const uint32_t off = TF32 ? mnmajor32_offset(row, c * 16u, w_lbo, 512u) : mnmajor_offset(row, c * 16u, w_lbo, 1024u);
        cp_async16(sw + off, wk + (size_t)row * w_row_bytes + c * 16u, true);
      }
    };

    OsWalk cur, pf;
    cur.init(t0, gsz, t1);
    pf = cur;
    int e[OS_PREFETCH];
#pragma unroll
    for (int d = 0; d < OS_PREFETCH; ++d) {
      e[d] = pf.tb < t1 ? load_entry(pf) : -1;
      pf.next(gsz, t1, p.k_vol);
    }
    int s = 0, n_load = -1, wb = 0;
    uint32_t ph = 0;
    while (cur.tb < t1 && ok) {
      int ent = e[0];
#pragma unroll
      for (int d = 0; d + 1 < OS_PREFETCH; ++d) e[d] = e[d + 1];
      e[OS_PREFETCH - 1] = pf.tb < t1 ? load_entry(pf) : -1;
      pf.next(gsz, t1, p.k_vol);
      if ((unsigned)ent >= (unsigned)p.n_in) {
        if (ent != -1) report_problem();  // an entry outside the tensor: treated as no neighbour, counted
        ent = -1;
      }
      if (cur.g == 0) {
        // a new offset: weight load number n_load goes to buffer n_load % n_wbuf, whose previous tenant was load
        // n_load - n_wbuf — wait until the MMA warp has reported that tenant's last MMA finished
        ++n_load;
        wb = (cfg.n_wbuf == 2) ? (n_load & 1) : 0;
        if (n_load >= cfg.n_wbuf) {
          const uint32_t use = (uint32_t)(cfg.n_wbuf == 2 ? (n_load >> 1) : n_load) - 1u;
          ok = g3_wait(&sh->w_free[wb], use & 1u, abort_flag);
          if (!ok) break;
        }
        load_weights(cur.k, wb);  // the first stage's barrier below also covers these copies
      }
      const uint8_t* rsrc[4];
      bool valid[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int g = __shfl_sync(0xffffffffu, ent, rs + 4 * j);
        valid[j] = g >= 0;
        rsrc[j] = src + (size_t)max(g, 0) * k_bytes + (size_t)pc * 16;
      }
      for (int kc = 0; kc < kch && ok; ++kc) {
        ok = g3_wait(&sh->empty[s], ph ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t st = smem_u32(sStage + (size_t)s * G3_STAGE_BYTES);
        if (kc * 128 + pc * 16 < k_bytes) {
#pragma unroll
          for (int j = 0; j < 4; ++j) cp_async16(st + a_dst[j], rsrc[j] + (size_t)kc * 128, valid[j]);
        }
        cp_async_arrive_noinc(smem_u32(&sh->full[s]));
        if (++s == n_stage) { s = 0; ph ^= 1u; }
      }
      cur.next(gsz, t1, p.k_vol);
    }
  } else if (warp == OS_MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc(TF32, false, true, OS_TILE, cfg.n_mma);
    const uint64_t a_desc0 = make_sdesc(smem_u32(sStage), 16u, 1024u);
    const uint64_t b_desc0 = make_sdesc(smem_u32(sW), (uint32_t)p.c_in * 128u, TF32 ? 512u : 1024u, TF32 ? 1u : 2u);
    const uint32_t b_kc_step = (uint32_t)EPR * 8u;        // one 128-byte K chunk further, in 16-byte units
    const uint32_t b_ks_step = (32u / ES) * 8u;           // one 32-byte MMA step further
    OsWalk cur;
    cur.init(t0, gsz, t1);
    int s = 0, n_load = -1, wb = 0, grp_i = 0, last_tb = t0;
    uint32_t ph = 0;
    // one lane runs the whole loop (waits, issue, commits); the other lanes wait at the end
    if (lane == 0)
    while (cur.tb < t1 && ok) {
      if (cur.tb != last_tb) { last_tb = cur.tb; ++grp_i; }
      if (cur.g == 0) {
        ++n_load;
        wb = (cfg.n_wbuf == 2) ? (n_load & 1) : 0;
      }
      if (cur.k == 0) {
        // first offset of the group: the accumulator must have been drained by the epilogue of the previous group
        ok = mbar_wait(smem_u32(&sh->tmem_empty[cur.g]), ((uint32_t)grp_i & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
      }
      const uint32_t d_tmem = tmem_base + (uint32_t)(cur.g * cfg.n_acc);
      const uint64_t b_desc_w = b_desc0 + (uint64_t)((uint32_t)wb * ((uint32_t)cfg.w_bytes >> 4));
      const bool last_k = cur.k == p.k_vol - 1, last_of_w = cur.g == cur.gv - 1;
      for (int kc = 0; kc < kch && ok; ++kc) {
        ok = mbar_wait(smem_u32(&sh->full[s]), ph, abort_flag);
        if (!ok) break;
        {
          fence_proxy_async();
          tc_fence_after();
          const uint64_t a_desc_s = a_desc0 + (uint64_t)((uint32_t)s * (G3_STAGE_BYTES >> 4));
          const uint64_t b_desc_kc = b_desc_w + (uint64_t)((uint32_t)kc * b_kc_step);
          const int n_ks = min(4, (k_bytes - kc * 128) >> 5);
          for (int ks = 0; ks < n_ks; ++ks)
            mma_ss<TF32>(d_tmem, a_desc_s + (uint64_t)(ks * 2), b_desc_kc + (uint64_t)((uint32_t)ks * b_ks_step), idesc,
                         (cur.k | kc | ks) != 0);
          mma_commit(smem_u32(&sh->empty[s]));
          if (kc == kch - 1) {
            if (last_k) mma_commit(smem_u32(&sh->tmem_full[cur.g]));
            if (last_of_w) mma_commit(smem_u32(&sh->w_free[wb]));
          }
        }
        if (++s == n_stage) { s = 0; ph ^= 1u; }
      }
      cur.next(gsz, t1, p.k_vol);
    }
    __syncwarp();
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3)
    // Warp q owns TMEM lanes 32 q .. 32 q + 31 = tile rows 32 q + lane.  16 accumulator columns at a time:
    // tcgen05.ld -> bias, ReLU, conversion -> the warp's patch -> eight consecutive lanes write 128 consecutive
    // bytes of one output row.
    const uint32_t row_bytes = (uint32_t)p.c_out * ES;
    constexpr uint32_t BLK_COLS = 128 / ES;
    uint8_t* dst = static_cast<uint8_t*>(p.dst);
    uint8_t* patch = sPatch + warp * 4096;
    const uint32_t sw7 = (uint32_t)(lane & 7);
    const uint32_t ch = (uint32_t)(lane & 7), rsub = (uint32_t)(lane >> 3);
    int grp_i = 0;
    for (int tb = t0; tb < t1 && ok; tb += gsz, ++grp_i) {
      const int gv = min(gsz, t1 - tb);
      for (int g = 0; g < gv && ok; ++g) {
        ok = g3_wait(&sh->tmem_full[g], (uint32_t)grp_i & 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const int row0 = (tb + g) * OS_TILE + 32 * warp;  // output row of this warp's lane 0
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(g * cfg.n_acc);
        for (uint32_t cb = 0; cb < row_bytes; cb += 128) {
          const uint32_t vb = min(128u, row_bytes - cb);  // bytes of this block that belong to the row
          const uint32_t col0 = cb / ES;
#pragma unroll
          for (uint32_t c0 = 0; c0 < BLK_COLS; c0 += 16) {
            if (c0 * ES >= vb) break;  // columns beyond the row (n_acc is the row rounded up to a whole block)
            uint32_t v[16];
            tmem_ld16(taddr + col0 + c0, v);
            tmem_ld_wait();
            float f[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) f[k] = __uint_as_float(v[k]);
            if (p.bias != nullptr) {
              if (TF32) {
                const float4* b4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.bias) + col0 + c0);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const float4 b = __ldg(b4 + k);
                  f[4 * k] += b.x; f[4 * k + 1] += b.y; f[4 * k + 2] += b.z; f[4 * k + 3] += b.w;
                }
              } else {
                const uint4* b4 = reinterpret_cast<const uint4*>(static_cast<const __half*>(p.bias) + col0 + c0);
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                  const uint4 b = __ldg(b4 + k);
                  const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                    f[8 * k + 2 * j] += t.x; f[8 * k + 2 * j + 1] += t.y;
                  }
                }
              }
            }
            if (p.relu) {
#pragma unroll
              for (int k = 0; k < 16; ++k) f[k] = fmaxf(f[k], 0.f);
            }
            if (TF32) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                *reinterpret_cast<uint4*>(patch + lane * 128 + (((uint32_t)(c0 / 4 + k) ^ sw7) << 4)) =
                    make_uint4(__float_as_uint(f[4 * k]), __float_as_uint(f[4 * k + 1]), __float_as_uint(f[4 * k + 2]), __float_as_uint(f[4 * k + 3]));
            } else {
              uint32_t h[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) h[k] = pack_half2(f[2 * k], f[2 * k + 1]);
              *reinterpret_cast<uint4*>(patch + lane * 128 + (((c0 / 8) ^ sw7) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
              *reinterpret_cast<uint4*>(patch + lane * 128 + (((c0 / 8 + 1) ^ sw7) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
            }
          }
          if (cb + 128 >= row_bytes) {
            // accumulator fully read: hand it back before the last rows go out
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->tmem_empty[g]));
          }
          __syncwarp();
          const bool ch_ok = (ch << 4) < vb;
#pragma unroll
          for (uint32_t u = 0; u < 8; ++u) {
            const uint32_t r = rsub + 4 * u;
            const int orow = row0 + (int)r;
            const uint4 v = *reinterpret_cast<const uint4*>(patch + r * 128 + ((ch ^ (r & 7)) << 4));
            if (orow < p.n_out && ch_ok) {
              uint8_t* o = dst + (size_t)orow * row_bytes + cb + (ch << 4);
              if (!p.accumulate) *reinterpret_cast<uint4*>(o) = v;
              else if (TF32) red_add_v4(reinterpret_cast<float*>(o), __uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
              else red_add_h8(reinterpret_cast<__half*>(o), v.x, v.y, v.z, v.w);
            }
          }
          __syncwarp();
        }
      }
    }
  }

  if (!ok && lane == 0) report_problem();
  cp_async_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == OS_MMA_WARP) tmem_dealloc(tmem_base, tmem_cols);
}

// 0 launched, 1 the shape has no plan or a pointer is not 16-byte aligned (there is no CUDA-core form of this
// kernel: the caller reports it), < 0 CUDA error
inline int launch_umma_osfwd(const OsParams& p, bool f16, cudaStream_t st, int sms, int max_smem) {
  if ((reinterpret_cast<uintptr_t>(p.src) | reinterpret_cast<uintptr_t>(p.weights) | reinterpret_cast<uintptr_t>(p.dst) |
       reinterpret_cast<uintptr_t>(p.bias)) & 15)
    return 1;
  G3Config cfg;
  if (!g3_plan(p.c_in, p.c_out, f16 ? 2 : 4, p.k_vol, max_smem, false, &cfg)) return 1;
  const int grid = p.n_tiles < sms ? p.n_tiles : sms;
  if (grid <= 0) return 0;
  if (f16) {
    static std::atomic<int> granted[64];
    if (int rc = ensure_smem(umma_osfwd_kernel<false>, max_smem, granted)) return rc;
    return launch_pdl(umma_osfwd_kernel<false>, grid, OS_THREADS, (size_t)cfg.smem, st, p, cfg) == cudaSuccess ? 0 : -1;
  }
  static std::atomic<int> granted[64];
  if (int rc = ensure_smem(umma_osfwd_kernel<true>, max_smem, granted)) return rc;
  return launch_pdl(umma_osfwd_kernel<true>, grid, OS_THREADS, (size_t)cfg.smem, st, p, cfg) == cudaSuccess ? 0 : -1;
}

}  // namespace fgms
