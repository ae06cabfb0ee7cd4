// Forward / dgrad on tcgen05, second design: every warp of the CTA takes part in every phase.
//
// The first design (umma_kernels.cuh) splits the CTA into five kinds of warps that hand work to each
// other through a dozen mbarrier rings.  Cycle traces showed its throughput limited by those
// hand-offs, not by any bandwidth.  This kernel keeps the same data path — 16-byte cp.async gathers
// straight into the 128-byte-swizzled tcgen05 operand layout, tcgen05.mma into tensor memory,
// tcgen05.ld -> shared-memory patch -> coalesced vector reds — but runs it as ONE software-pipelined
// loop executed by all 8 warps, with the asynchrony supplied by the hardware queues instead of by
// polling warps:
//
//   iteration t :  [wait MMA(t-1)]  issue gathers of tile t+1  |  wait gathers of tile t, sync
//                  thread 0 issues the MMAs of tile t (async)  |  all warps drain + scatter tile t-1
//                  stash the map entries of tile t+2, start loading those of tile t+3
//
// so that the gathers of tile t+1, the MMAs of tile t and the scatter of tile t-1 overlap.  Two
// gather buffers, two weight buffers (no stall when the kernel offset changes), two TMEM
// accumulators.  Several CTAs share an SM when shared memory and TMEM allow (small channel counts).
#pragma once

#include "common.cuh"
#include "umma.cuh"

namespace fgms {

constexpr int G2_THREADS = 256;
constexpr int G2_TILE_M = 128;
constexpr int G2_IDX_RING = 4;

struct G2Shared {
  uint64_t mma_done[2];        // tcgen05.commit of the tile that used accumulator / gather buffer b
  uint32_t tmem_base;
  int abort_flag;
  int idx_g[G2_IDX_RING][G2_TILE_M];  // raw gather-map entries of a tile
  int idx_s[G2_IDX_RING][G2_TILE_M];  // raw scatter-map entries
};
constexpr int G2_SHARED_BYTES = (sizeof(G2Shared) + 255) & ~255;

struct G2Config {
  int a_tile_bytes;   // kch * 16 KB
  int w_bytes;        // k_dim * n_dim * elem
  int n_wbuf;         // 1 or 2
  int patch_bytes;    // 128 rows x min(256, row bytes)
};

template <bool TF32, bool TRANS_W>
__global__ void __launch_bounds__(G2_THREADS) umma_gms2_kernel(GmsParams p, G2Config cfg) {
  using namespace umma;
  constexpr int ES = TF32 ? 4 : 2;
  constexpr int EPR = 128 / ES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sW = smem;                                   // n_wbuf weight operands
  uint8_t* sA = sW + (size_t)cfg.n_wbuf * cfg.w_bytes;  // 2 gathered tiles
  uint8_t* sPatch = sA + 2 * (size_t)cfg.a_tile_bytes;
  G2Shared* sh = reinterpret_cast<G2Shared*>(sPatch + cfg.patch_bytes);
  int* tile_start = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(sh) + G2_SHARED_BYTES);  // [k_vol + 2]
  int* kpos_s = tile_start + p.k_vol + 2;                                                        // [k_vol + 1]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_seg = p.k_vol + 1;
  const int kch = p.k_dim / EPR;
  const uint32_t row_bytes = (uint32_t)p.n_dim * ES;
  volatile int* abort_flag = &sh->abort_flag;

  if (tid == 0) {
    mbar_init(smem_u32(&sh->mma_done[0]), 1);
    mbar_init(smem_u32(&sh->mma_done[1]), 1);
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  for (int s = tid; s <= p.k_vol; s += G2_THREADS) kpos_s[s] = __ldg(p.kpos + s);
  build_tile_table(G2_TILE_M, p.kpos, p.k_vol, p.dense_rows, tile_start);  // syncs the CTA
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2u * p.n_dim) tmem_cols <<= 1;
  if (warp == 0) {
    tmem_alloc(smem_u32(&sh->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);
  const int n_tiles = t1 - t0;

  // ---- per-tile bookkeeping (all from shared memory) ----
  struct Tile { int seg, base, cnt, widx; bool dense; };
  auto tile_info = [&](int t) {
    Tile ti;
    ti.seg = find_segment(tile_start, n_seg, t);
    const int lt = t - tile_start[ti.seg];
    ti.dense = ti.seg == p.k_vol;
    const int seg_base = ti.dense ? 0 : kpos_s[ti.seg];
    const int seg_cnt = ti.dense ? p.dense_rows : (kpos_s[ti.seg + 1] - seg_base);
    ti.base = seg_base + lt * G2_TILE_M;
    ti.cnt = min(G2_TILE_M, seg_cnt - lt * G2_TILE_M);
    ti.widx = ti.dense ? p.dense_weight : ti.seg;
    return ti;
  };
  // thread tid < 128 fetches the gather entry of row tid, thread tid >= 128 the scatter entry of row tid - 128
  auto load_entry = [&](int t) -> int {
    if (t >= t1) return -1;
    const Tile ti = tile_info(t);
    const int row = tid & 127;
    if (row >= ti.cnt) return -1;
    if (ti.dense) return ti.base + row;
    return __ldg((tid < 128 ? p.gather_map : p.scatter_map) + ti.base + row);
  };
  auto stash_entry = [&](int t, int v) {
    if (tid < 128) sh->idx_g[t & (G2_IDX_RING - 1)][tid] = v;
    else sh->idx_s[t & (G2_IDX_RING - 1)][tid - 128] = v;
  };
  // a pair is used only if both its entries are inside the tensors
  auto pair_ok = [&](int g, int s) { return (unsigned)g < (unsigned)p.n_gather && (unsigned)s < (unsigned)p.n_scatter; };

  // ---- gather role of this thread: chunk pc of rows prow + 32 q ----
  const int prow = tid >> 3, pc = tid & 7;
  const uint32_t a_dst0 = (uint32_t)(prow >> 3) * 1024u + (uint32_t)(prow & 7) * 128u + (uint32_t)((pc ^ (prow & 7)) << 4);
  const uint8_t* src = static_cast<const uint8_t*>(p.src);
  const uint8_t* wts = static_cast<const uint8_t*>(p.weights);
  const size_t src_row_bytes = (size_t)p.k_dim * ES;
  const uint32_t w_row_bytes = (uint32_t)p.c_out * ES;

  auto load_weights = [&](int widx, int wb) {
    const uint8_t* wk = wts + (size_t)widx * p.c_in * p.c_out * ES;
    const uint32_t sw = smem_u32(sW + (size_t)wb * cfg.w_bytes);
    if (!TRANS_W) {
      const int cpr = p.n_dim * ES / 16, total = p.k_dim * cpr;
      const uint32_t lbo = (uint32_t)p.k_dim * 128u;
      for (int e = tid; e < total; e += G2_THREADS) {
        const uint32_t row = e / cpr, c = e % cpr;
        const uint32_t off = TF32 ? mnmajor32_offset(row, c * 16u, lbo, 512u) : mnmajor_offset(row, c * 16u, lbo, 1024u);
        cp_async16(sw + off, wk + (size_t)row * w_row_bytes + c * 16u, true);
      }
    } else {
      const int cpr = p.k_dim * ES / 16, total = p.n_dim * cpr;
      for (int e = tid; e < total; e += G2_THREADS) {
        const uint32_t row = e / cpr, c = e % cpr;
        cp_async16(sw + kmajor_offset(row, c * 16u, p.n_dim), wk + (size_t)row * w_row_bytes + c * 16u, true);
      }
    }
  };
  // gathers of local tile i into buffer i & 1 (map entries come from the shared-memory ring, which is
  // indexed by the global tile number; every double buffer is indexed by the LOCAL tile number)
  auto issue_gather = [&](int i) {
    const int slot = (t0 + i) & (G2_IDX_RING - 1);
    const uint32_t st = smem_u32(sA + (size_t)(i & 1) * cfg.a_tile_bytes) + a_dst0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int row = prow + 32 * q;
      const int g = sh->idx_g[slot][row], s = sh->idx_s[slot][row];
      const bool valid = pair_ok(g, s);
      if (!valid && pc == 0 && (g != -1 || s != -1)) report_problem();  // entry outside the tensors: pair skipped, counted once
      const uint8_t* rsrc = valid ? src + (size_t)g * src_row_bytes + (size_t)pc * 16 : src;
      for (int kc = 0; kc < kch; ++kc)
        cp_async16(st + (uint32_t)q * 4096u + (uint32_t)kc * 16384u, rsrc + (valid ? (size_t)kc * 128 : 0), valid);
    }
  };
  // thread 0: the MMAs of local tile i
  const uint32_t idesc = make_idesc(TF32, false, !TRANS_W, G2_TILE_M, p.n_dim);
  auto issue_mma = [&](int i, int wb) {
    const uint32_t sa = smem_u32(sA + (size_t)(i & 1) * cfg.a_tile_bytes);
    const uint32_t sw = smem_u32(sW + (size_t)wb * cfg.w_bytes);
    const uint32_t d_tmem = tmem_base + (uint32_t)(i & 1) * p.n_dim;
    for (int kc = 0; kc < kch; ++kc) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t a_desc = make_sdesc(sa + (uint32_t)kc * 16384u + ks * 32u, 16u, 1024u);
        uint64_t b_desc;
        if (!TRANS_W) {
          const uint32_t k_row = (uint32_t)kc * EPR + (uint32_t)ks * (32u / ES);
          b_desc = make_sdesc(sw + k_row * 128u, (uint32_t)p.k_dim * 128u, TF32 ? 512u : 1024u, TF32 ? 1u : 2u);
        } else {
          b_desc = make_sdesc(sw + (uint32_t)kc * ((uint32_t)p.n_dim * 128u) + ks * 32u, 16u, 1024u);
        }
        mma_ss<TF32>(d_tmem, a_desc, b_desc, idesc, (kc | ks) != 0);
      }
    }
    mma_commit(smem_u32(&sh->mma_done[i & 1]));
  };
  // all warps: accumulator of local tile i -> destination rows.  Warp (q, h): TMEM lanes 32 q .. 32 q + 31
  // (a warp may only read the lane quarter given by its index mod 4) and half h of every 256-byte block.
  uint8_t* dst = static_cast<uint8_t*>(p.dst);
  const int q4 = warp & 3, hh = warp >> 2;
  uint8_t* patch = sPatch + warp * 4096;  // 32 rows x 128 bytes, private to the warp
  auto epilogue = [&](int i) {
    const int slot = (t0 + i) & (G2_IDX_RING - 1);
    const int row = 32 * q4 + lane;
    const int eg = sh->idx_g[slot][row], es = sh->idx_s[slot][row];
    const int srow = pair_ok(eg, es) ? es : -1;
    const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(i & 1) * p.n_dim;
    const uint32_t sw7 = (uint32_t)(lane & 7);
    for (uint32_t cb = 0; cb < row_bytes; cb += 256) {
      const uint32_t half = min(256u, row_bytes - cb) >> 1;  // bytes of this block handled by this warp: 128 or 64
      const uint32_t my0 = cb + hh * half;
      const uint32_t ncol = half / ES, col0 = my0 / ES;
      for (uint32_t c0 = 0; c0 < ncol; c0 += 32) {
        uint32_t v0[16], v1[16];
        const bool two = c0 + 16 < ncol;
        tmem_ld16(taddr + col0 + c0, v0);
        if (two) tmem_ld16(taddr + col0 + c0 + 16, v1);
        tmem_ld_wait();
        if (TF32) {
          const uint32_t ch0 = c0 / 4;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            *reinterpret_cast<uint4*>(patch + lane * 128 + (((ch0 + k) ^ sw7) << 4)) = make_uint4(v0[4 * k], v0[4 * k + 1], v0[4 * k + 2], v0[4 * k + 3]);
            if (two) *reinterpret_cast<uint4*>(patch + lane * 128 + (((ch0 + 4 + k) ^ sw7) << 4)) = make_uint4(v1[4 * k], v1[4 * k + 1], v1[4 * k + 2], v1[4 * k + 3]);
          }
        } else {
          const uint32_t ch0 = c0 / 8;
          uint32_t h[16];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            h[k] = pack_half2(__uint_as_float(v0[2 * k]), __uint_as_float(v0[2 * k + 1]));
            h[8 + k] = pack_half2(__uint_as_float(v1[2 * k]), __uint_as_float(v1[2 * k + 1]));
          }
          *reinterpret_cast<uint4*>(patch + lane * 128 + (((ch0 + 0) ^ sw7) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<uint4*>(patch + lane * 128 + (((ch0 + 1) ^ sw7) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
          if (two) {
            *reinterpret_cast<uint4*>(patch + lane * 128 + (((ch0 + 2) ^ sw7) << 4)) = make_uint4(h[8], h[9], h[10], h[11]);
            *reinterpret_cast<uint4*>(patch + lane * 128 + (((ch0 + 3) ^ sw7) << 4)) = make_uint4(h[12], h[13], h[14], h[15]);
          }
        }
      }
      __syncwarp();
      const uint32_t cpr = half >> 4;   // 16-byte chunks per row in my part: 8 or 4
      const uint32_t rpi = 32 / cpr;    // rows per warp-wide instruction: 4 or 8
      const uint32_t ch = lane % cpr, rsub = lane / cpr;
      uint8_t* dcol = dst + my0 + (ch << 4);
#pragma unroll 4
      for (uint32_t r0 = 0; r0 < 32; r0 += rpi) {
        const uint32_t r = r0 + rsub;
        const int sr = __shfl_sync(0xffffffffu, srow, r);
        const uint4 v = *reinterpret_cast<const uint4*>(patch + r * 128 + ((ch ^ (r & 7)) << 4));
        if (sr >= 0) {
          uint8_t* o = dcol + (size_t)sr * row_bytes;
          if (TF32) red_add_v4(reinterpret_cast<float*>(o), __uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
          else red_add_h8(reinterpret_cast<__half*>(o), v.x, v.y, v.z, v.w);
        }
      }
      __syncwarp();
    }
    tc_fence_before();
  };
  auto wait_mma = [&](int i) -> bool {  // MMAs of local tile i have finished
    int ok = 1;
    if (lane == 0) ok = mbar_wait(smem_u32(&sh->mma_done[i & 1]), (uint32_t)(i >> 1) & 1u, abort_flag) ? 1 : 0;
    __syncwarp();
    ok = __shfl_sync(0xffffffffu, ok, 0);
    tc_fence_after();
    return ok != 0;
  };

  // ---- the pipelined loop ----
  bool ok = true;
  int cur_w = -1, cur_wb = 0, wb_of[2] = {0, 0};
  auto prefetch_tile = [&](int i) {  // weights (if they change) + gathers of local tile i, one cp.async group
    const Tile ti = tile_info(t0 + i);
    if (ti.widx != cur_w) {
      cur_wb = (cfg.n_wbuf == 2) ? (cur_wb ^ 1) : 0;
      load_weights(ti.widx, cur_wb);
      cur_w = ti.widx;
    }
    wb_of[i & 1] = cur_wb;
    issue_gather(i);
    cp_async_commit();
  };

  if (n_tiles > 0) {
    stash_entry(t0, load_entry(t0));
    stash_entry(t0 + 1, load_entry(t0 + 1));
    int pend = load_entry(t0 + 2);
    __syncthreads();
    prefetch_tile(0);
    for (int i = 0; i < n_tiles && ok; ++i) {
      // 1. the MMAs of tile i-1 are done: its gather buffer (the one tile i+1 uses) is free, its accumulator is ready
      if (i >= 1) ok = wait_mma(i - 1);
      if (!ok) break;
      // 2. start the gathers of tile i+1 (with a single weight buffer a weight change has to wait for MMA(i))
      const bool have_next = i + 1 < n_tiles;
      bool next_issued = false;
      if (have_next && (cfg.n_wbuf == 2 || tile_info(t0 + i + 1).widx == cur_w)) {
        prefetch_tile(i + 1);
        next_issued = true;
      }
      // 3. the gathers of tile i have landed (every thread waits for its own, then the CTA meets)
      if (next_issued) cp_async_wait<1>(); else cp_async_wait<0>();
      fence_proxy_async();
      __syncthreads();
      // 4. MMAs of tile i
      if (tid == 0) {
        tc_fence_after();
        issue_mma(i, wb_of[i & 1]);
      }
      // 5. drain + scatter tile i-1 while the tensor core works on tile i
      if (i >= 1) epilogue(i - 1);
      // 6. map entries: park those of tile i+2, start loading those of tile i+3
      stash_entry(t0 + i + 2, pend);
      pend = load_entry(t0 + i + 3);
      if (have_next && !next_issued) {
        ok = wait_mma(i);
        if (ok) prefetch_tile(i + 1);
      }
      __syncthreads();
    }
    if (ok) ok = wait_mma(n_tiles - 1);
    if (ok) epilogue(n_tiles - 1);
  }

  if (!ok && lane == 0) report_problem();
  cp_async_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
}

// host launcher: 0 launched, 1 shape does not fit (caller falls back), < 0 CUDA error
template <typename K>
inline int g2_ensure_smem(K kernel, int bytes, int slot) {
  static int granted[4][64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (granted[slot][dev] >= bytes) return 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -1;
  granted[slot][dev] = bytes;
  return 0;
}

inline int launch_umma_gms2(const GmsParams& p, bool trans, bool f16, cudaStream_t st, int sms, int max_smem) {
  const int es = f16 ? 2 : 4;
  if ((reinterpret_cast<uintptr_t>(p.src) | reinterpret_cast<uintptr_t>(p.weights) | reinterpret_cast<uintptr_t>(p.dst)) & 15) return 1;
  G2Config cfg;
  cfg.a_tile_bytes = (p.k_dim * es / 128) * 16384;
  cfg.w_bytes = p.k_dim * p.n_dim * es;
  cfg.patch_bytes = 8 * 4096;
  const int table = ((2 * p.k_vol + 3) * 4 + 15) & ~15;
  const int fixed = 1024 + cfg.patch_bytes + G2_SHARED_BYTES + table + 2 * cfg.a_tile_bytes;
  cfg.n_wbuf = (fixed + 2 * cfg.w_bytes <= max_smem) ? 2 : 1;
  const int smem = fixed + cfg.n_wbuf * cfg.w_bytes;
  if (smem > max_smem) return 1;
  // CTAs per SM: limited by shared memory (227 KB per SM, 1 KB reserved per CTA) and by the 512 TMEM columns
  int tmem_cols = 32;
  while (tmem_cols < 2 * p.n_dim) tmem_cols <<= 1;
  int rc;
  auto ctas_per_sm = [&](auto kernel) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, G2_THREADS, (size_t)smem) != cudaSuccess || n < 1) n = 1;
    if (n > 512 / tmem_cols) n = 512 / tmem_cols;  // every resident CTA holds its TMEM columns for its whole life
    return n < 1 ? 1 : n;
  };
  if (f16) {
    if (trans) { rc = g2_ensure_smem(umma_gms2_kernel<false, true>, max_smem, 0); if (rc) return rc; umma_gms2_kernel<false, true><<<sms * ctas_per_sm(umma_gms2_kernel<false, true>), G2_THREADS, smem, st>>>(p, cfg); }
    else       { rc = g2_ensure_smem(umma_gms2_kernel<false, false>, max_smem, 1); if (rc) return rc; umma_gms2_kernel<false, false><<<sms * ctas_per_sm(umma_gms2_kernel<false, false>), G2_THREADS, smem, st>>>(p, cfg); }
  } else {
    if (trans) { rc = g2_ensure_smem(umma_gms2_kernel<true, true>, max_smem, 2); if (rc) return rc; umma_gms2_kernel<true, true><<<sms * ctas_per_sm(umma_gms2_kernel<true, true>), G2_THREADS, smem, st>>>(p, cfg); }
    else       { rc = g2_ensure_smem(umma_gms2_kernel<true, false>, max_smem, 3); if (rc) return rc; umma_gms2_kernel<true, false><<<sms * ctas_per_sm(umma_gms2_kernel<true, false>), G2_THREADS, smem, st>>>(p, cfg); }
  }
  return 0;
}

}  // namespace fgms
