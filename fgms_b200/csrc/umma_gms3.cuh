// Forward / dgrad on tcgen05, warp-specialised with private hand-offs only.
//
//   out[scatter[j]] += src[gather[j]] . W_k        for the pairs j of every offset k
//
// One persistent CTA per SM walks a contiguous range of 128-pair tiles.  Seventeen warps, three roles,
// and the only things that cross between roles are mbarrier phases:
//
//   producers (8 warps)  fetch their rows' map entries straight from global memory two tiles ahead,
//                        gather feature rows with 16-byte cp.async into a ring of 16 KB stages (one
//                        128-byte K chunk of 128 rows each, K-major SWIZZLE_128B) and, when the offset
//                        changes, the next weight matrix into the other of two weight buffers;
//   MMA warp             one lane issues tcgen05.mma per stage, commits the stage back to the producers
//                        and the finished accumulator (two TMEM buffers) to the epilogue;
//   epilogue (8 warps)   two warps per TMEM lane quarter, each owning half of every 256-byte block of the
//                        output row: tcgen05.ld -> convert -> a 4 KB patch private to the warp -> 16-byte
//                        vector reds with consecutive lanes on consecutive addresses of one row.  The map
//                        entries of its 32 rows come from global memory two tiles ahead as well.
//
// Every role recomputes the (cheap) tile bookkeeping from the tile table in shared memory, so there is
// no index ring and no patch hand-off.  All waits are bounded; a wait that runs out sets the CTA's
// abort flag, every role leaves its loop, in-flight copies are awaited and TMEM is freed.
#pragma once
#include <atomic>

#include "common.cuh"
#include "umma.cuh"

namespace fgms {

// Shapes the tensor-core kernels take: both channel counts multiples of 16, at most 256.  A gathered row
// then is a whole number of 32-byte MMA steps and at least two 16-byte chunks; rows shorter than a
// 128-byte swizzle span (fp16 C = 16 / 32 / 48, tf32 C = 16) fill the front of a span and the rest of
// the span is never read.  Whether a shape also fits shared memory is decided by g3_plan / w3_plan.
inline bool umma_supported(int c_in, int c_out, int elem_bytes) {
  (void)elem_bytes;
  return c_in % 16 == 0 && c_out % 16 == 0 && c_in >= 16 && c_out >= 16 && c_in <= 256 && c_out <= 256;
}

constexpr int G3_TILE_M = 128;
constexpr int G3_EPI_WARPS = 8;
constexpr int G3_MMA_WARP = 8;
constexpr int G3_PROD_WARP0 = 9;
constexpr int G3_PROD_WARPS = 8;
constexpr int G3_PROD_THREADS = G3_PROD_WARPS * 32;
constexpr int G3_THREADS = (G3_PROD_WARP0 + G3_PROD_WARPS) * 32;  // 544
constexpr int G3_STAGE_BYTES = 16384;
constexpr int G3_MAX_STAGES = 8;
constexpr int G3_PATCH_BYTES = G3_EPI_WARPS * 4096;
// Map entries are prefetched two tiles ahead with 4-byte cp.async into a ring private to each warp (each
// lane writes and later reads only its own word, so no synchronisation is involved): a load into a
// register would have to be waited for as soon as the register is copied, one tile later.
constexpr int G3_RING_SLOTS = 4;
constexpr int G3_RING_BYTES = (G3_PROD_WARPS + 2 * G3_EPI_WARPS) * G3_RING_SLOTS * 128;

struct G3Shared {
  uint64_t full[G3_MAX_STAGES];   // stage landed (one hardware arrival per producer thread)
  uint64_t empty[G3_MAX_STAGES];  // stage consumed (tcgen05.commit)
  uint64_t tmem_full[4];          // accumulator finished (tcgen05.commit)
  uint64_t tmem_empty[4];         // accumulator drained (one arrival per warp of the group that owns it)
  uint64_t w_free[2];             // every MMA that reads this weight buffer has finished (tcgen05.commit)
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int G3_SHARED_BYTES = (sizeof(G3Shared) + 15) & ~15;

struct G3Config {
  int n_stage;  // gather stages in the ring
  int n_wbuf;   // weight buffers: 2 when they fit, else 1 (a change of offset then drains the MMAs)
  int w_bytes;  // one weight operand in its tcgen05 layout (whole 128-byte spans)
  int n_tbuf;   // TMEM accumulators: 4 when 4 x n_acc columns fit in the 512, else 2
  int tbuf_shift;  // log2(n_tbuf)
  int kch;      // 128-byte K chunks (= stages) per tile: ceil(k_dim * elem / 128)
  int n_acc;    // TMEM columns per accumulator: n_dim rounded up to whole 128-byte blocks of the output row
  int n_mma;    // N of the MMA: n_acc for the MN-major weight operand (forward), n_dim for the K-major one (dgrad)
  int smem;     // dynamic shared memory of the launch
};

// Every lane probes the barrier itself (one broadcast read per probe, and each lane's own acquire orders its later
// reads); one vote makes the outcome the warp's, so that a wait that ran out takes the whole warp out of its loop.
__device__ __forceinline__ bool g3_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = umma::mbar_wait(umma::smem_u32(bar), parity, abort_flag);
  return __all_sync(0xffffffffu, ok) != 0;
}

// Walks consecutive tiles of the tile table without searching: the segment only ever moves forward.
struct G3Walk {
  int t, seg, seg_first, seg_end;  // tile, its segment, the segment's first tile and one past its last
  __device__ __forceinline__ void init(const int* tile_start, int n_seg, int t_) {
    t = t_;
    seg = find_segment(tile_start, n_seg, t_);
    seg_first = tile_start[seg];
    seg_end = tile_start[seg + 1];
  }
  __device__ __forceinline__ void next(const int* tile_start, int n_seg) {
    ++t;
    while (t >= seg_end && seg + 1 < n_seg) {
      ++seg;
      seg_first = seg_end;
      seg_end = tile_start[seg + 1];
    }
  }
};
struct G3Tile { int base, cnt, widx; bool dense; };
__device__ __forceinline__ G3Tile g3_tile(const G3Walk& w, const GmsParams& p, const int* kpos_s) {
  G3Tile ti;
  const int lt = w.t - w.seg_first;
  ti.dense = w.seg == p.k_vol;
  const int seg_base = ti.dense ? 0 : kpos_s[w.seg];
  const int seg_cnt = ti.dense ? p.dense_rows : (kpos_s[w.seg + 1] - seg_base);
  ti.base = seg_base + lt * G3_TILE_M;
  ti.cnt = min(G3_TILE_M, seg_cnt - lt * G3_TILE_M);
  ti.widx = ti.dense ? p.dense_weight : w.seg;
  return ti;
}

// the weight matrix of the walk's tile (needs no table access)
__device__ __forceinline__ int g3_widx(const G3Walk& w, const GmsParams& p) { return w.seg == p.k_vol ? p.dense_weight : w.seg; }

// FULL: both row lengths are whole 128-byte spans (the large-channel layers).  Every per-chunk guard below is
// then a compile-time constant; the hot loops of that instantiation carry no test the short-row shapes need.
template <bool TF32, bool TRANS_W, bool FULL>
__global__ void __launch_bounds__(G3_THREADS, 1) umma_gms3_kernel(GmsParams p, G3Config cfg) {
  using namespace umma;
  constexpr int ES = TF32 ? 4 : 2;
  constexpr int EPR = 128 / ES;  // elements per 128-byte span
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sW = smem;                                      // n_wbuf weight operands
  uint8_t* sStage = sW + (size_t)cfg.n_wbuf * cfg.w_bytes;  // gather ring
  uint8_t* sPatch = sStage + (size_t)cfg.n_stage * G3_STAGE_BYTES;
  uint8_t* sRing = sPatch + G3_PATCH_BYTES;
  G3Shared* sh = reinterpret_cast<G3Shared*>(sRing + G3_RING_BYTES);
  int* tile_start = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(sh) + G3_SHARED_BYTES);  // [k_vol + 2]
  int* kpos_s = tile_start + p.k_vol + 2;                                                        // [k_vol + 1]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_seg = p.k_vol + 1;
  const int kch = cfg.kch;                   // 128-byte K chunks per gathered row (the last one may be partly filled)
  const int k_bytes = p.k_dim * ES;          // bytes of a gathered row: a multiple of 32
  const int n_stage = cfg.n_stage;
  volatile int* abort_flag = &sh->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < n_stage; ++s) {
      mbar_init(smem_u32(&sh->full[s]), G3_PROD_THREADS);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(smem_u32(&sh->tmem_full[b]), 1);
      mbar_init(smem_u32(&sh->tmem_empty[b]), G3_EPI_WARPS / 2);
    }
    mbar_init(smem_u32(&sh->w_free[0]), 1);
    mbar_init(smem_u32(&sh->w_free[1]), 1);
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  // TMEM allocation overlaps the first global loads below
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)(cfg.n_tbuf * cfg.n_acc)) tmem_cols <<= 1;
  if (warp == G3_MMA_WARP) {
    tmem_alloc(smem_u32(&sh->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  // everything above touches no global memory; from here on the previous kernel's results may be needed
  griddep_wait();
  griddep_launch_dependents();
  build_tile_table(G3_TILE_M, p.kpos, p.pairs, p.k_vol, p.dense_rows, kpos_s, tile_start);  // syncs the CTA
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);
  bool ok = true;
  // a pair is used only if both its entries are inside the tensors
  auto pair_ok = [&](int g, int s) { return (unsigned)g < (unsigned)p.n_gather && (unsigned)s < (unsigned)p.n_scatter; };

  if (t0 >= t1) {
    // nothing for this CTA
  } else if (warp >= G3_PROD_WARP0) {
    // ------------------------------------------------------------------ producers
    // Warp pw owns tile rows [16 pw, 16 pw + 16).  Lanes 0-15 fetch those rows' gather entries, lanes
    // 16-31 their scatter entries (needed to skip pairs whose destination is outside the tensor).
    const int pw = warp - G3_PROD_WARP0;
    const int tp = tid - G3_PROD_WARP0 * 32;
    // `lpr` lanes share a row, one 16-byte chunk each: 8 for rows of a whole span or more, 4 / 2 for 64- /
    // 32-byte rows, so that short rows still keep every lane busy.  This thread copies chunk pc of the rows
    // 16 pw + rsub + rpp j, j < n_pass.
    const int lpr = (FULL || k_bytes > 64) ? 8 : (k_bytes > 32 ? 4 : 2);
    const int rpp = 32 / lpr, n_pass = FULL ? 4 : 16 / rpp;  // rows per warp-wide copy: 4 / 8 / 16; copies per tile: 4 / 2 / 1
    const int pc = lane % lpr, rsub = lane / lpr;
    const uint8_t* src = static_cast<const uint8_t*>(p.src);
    const uint8_t* wts = static_cast<const uint8_t*>(p.weights);
    const size_t src_row_bytes = (size_t)k_bytes;
    const uint32_t w_row_bytes = (uint32_t)p.c_out * ES;
    uint32_t a_dst[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t r = (uint32_t)(16 * pw + rsub + rpp * j) & 127u;
      a_dst[j] = (r >> 3) * 1024u + (r & 7u) * 128u + (((uint32_t)pc ^ (r & 7u)) << 4);
    }
    const uint32_t ring = smem_u32(sRing) + (uint32_t)(pw * G3_RING_SLOTS * 128 + lane * 4);  // this lane's word of slot 0
    auto fetch_entry = [&](const G3Walk& w, int slot) {
      const G3Tile ti = g3_tile(w, p, kpos_s);
      const int row = 16 * pw + (lane & 15);
      const uint32_t dst = ring + (uint32_t)slot * 128u;
      if (row < ti.cnt && !ti.dense) cp_async4(dst, (lane < 16 ? p.gather_map : p.scatter_map) + ti.base + row);
      else st_shared_i32(dst, row < ti.cnt ? ti.base + row : -1);
    };
    // Weight matrix -> operand layout.  The matrix is `w_rows` rows of `cpr` 16-byte chunks; when cpr divides the
    // number of producer threads every thread keeps one chunk column and strides over rows (no division in the loop).
    const int w_rows = p.c_in;             // rows of W_k in global memory: n_dim of them for dgrad, k_dim for forward
    const int cpr = p.c_out * ES / 16;     // 16-byte chunks per row
    const bool cpr_divides = (G3_PROD_THREADS % cpr) == 0;
    const uint32_t w_c = cpr_divides ? (uint32_t)(tp % cpr) : 0u;
    const int w_r0 = cpr_divides ? tp / cpr : 0, w_rstep = cpr_divides ? G3_PROD_THREADS / cpr : 0;
    const uint32_t w_lbo = (uint32_t)p.k_dim * 128u;
    auto w_offset = [&](uint32_t row, uint32_t c) -> uint32_t {
      if (TRANS_W) return kmajor_offset(row, c * 16u, p.n_dim);  // rows = output index: K-major operand
      return TF32 ? mnmajor32_offset(row, c * 16u, w_lbo, 512u) : mnmajor_offset(row, c * 16u, w_lbo, 1024u);  // rows = contraction index: MN-major
    };
    auto load_weights = [&](int widx, int wb) {
      const uint8_t* wk = wts + (size_t)widx * p.c_in * p.c_out * ES;
      const uint32_t sw = smem_u32(sW + (size_t)wb * cfg.w_bytes);
      if (cpr_divides) {
        const uint8_t* col = wk + w_c * 16u;
        for (int row = w_r0; row < w_rows; row += w_rstep)
          cp_async16(sw + w_offset((uint32_t)row, w_c), col + (size_t)row * w_row_bytes, true);
      } else {
        const int total = w_rows * cpr;
        for (int e = tp; e < total; e += G3_PROD_THREADS) {
          const uint32_t row = e / cpr, c = e % cpr;
          cp_async16(sw + w_offset(row, c), wk + (size_t)row * w_row_bytes + c * 16u, true);
        }
      }
    };

    G3Walk cur, pf;
    cur.init(tile_start, n_seg, t0);
    pf = cur;
    fetch_entry(pf, 0);
    cp_async_commit();
    pf.next(tile_start, n_seg);
    if (pf.t < t1) fetch_entry(pf, 1);
    cp_async_commit();
    pf.next(tile_start, n_seg);
    int s = 0;
    uint32_t ph = 0;          // stage and its phase
    int cur_w = -1, n_load = -1, wb = 0;

    for (int t = t0; t < t1 && ok; ++t) {
      if (pf.t < t1) fetch_entry(pf, (t - t0 + 2) & (G3_RING_SLOTS - 1));
      cp_async_commit();  // also closes the group of the previous tile's gathers
      pf.next(tile_start, n_seg);
      const G3Tile ti = g3_tile(cur, p, kpos_s);
      if (ti.widx != cur_w) {
        // weight load number n_load goes to buffer n_load % n_wbuf, whose previous tenant was load
        // n_load - n_wbuf: wait until the MMA warp has reported that tenant's last MMA finished
        ++n_load;
        wb = (cfg.n_wbuf == 2) ? (n_load & 1) : 0;
        if (n_load >= cfg.n_wbuf) {
          const uint32_t use = (uint32_t)(cfg.n_wbuf == 2 ? (n_load >> 1) : n_load) - 1u;
          ok = g3_wait(&sh->w_free[wb], use & 1u, abort_flag);
          if (!ok) break;
        }
        cur_w = ti.widx;
        // issued before the wait for this tile's map entries; the first stage's barrier below also covers these copies
        load_weights(ti.widx, wb);
      }
      cp_async_wait<2>();  // everything older than the last two groups has landed: this tile's entries have
      const int e0 = ld_shared_i32(ring + (uint32_t)((t - t0) & (G3_RING_SLOTS - 1)) * 128u);
      // lanes 0-15 hold gather entries, lanes 16-31 the scatter entries of the same rows: settle once per
      // pair whether it is used, then one shuffle per row hands out the gather entry (-1: zero-fill)
      const int other = __shfl_xor_sync(0xffffffffu, e0, 16);
      const int g_own = lane < 16 ? e0 : other, s_own = lane < 16 ? other : e0;
      const bool okp = pair_ok(g_own, s_own);
      if (!okp && lane < 16 && (g_own != -1 || s_own != -1)) report_problem();  // entry outside the tensors: pair skipped, counted once
      const int ev = okp ? g_own : -1;
      const uint8_t* rsrc[4];
      bool valid[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int g = __shfl_sync(0xffffffffu, ev, (rsub + rpp * j) & 15);
        valid[j] = g >= 0 && (FULL || j < n_pass);
        rsrc[j] = src + (size_t)max(g, 0) * src_row_bytes + (size_t)pc * 16;
      }
      for (int kc = 0; kc < kch && ok; ++kc) {
        ok = g3_wait(&sh->empty[s], ph ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t st = smem_u32(sStage + (size_t)s * G3_STAGE_BYTES);
        if (FULL || kc * 128 + pc * 16 < k_bytes) {  // the last chunk of a row that is no whole number of spans is partly filled
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (FULL || j < n_pass) cp_async16(st + a_dst[j], rsrc[j] + (size_t)kc * 128, valid[j]);
        }
        // the stage's barrier hears from this thread when everything it has issued so far has landed
        cp_async_arrive_noinc(smem_u32(&sh->full[s]));
        if (++s == n_stage) { s = 0; ph ^= 1u; }
      }
      cur.next(tile_start, n_seg);
    }
  } else if (warp == G3_MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc(TF32, false, !TRANS_W, G3_TILE_M, cfg.n_mma);
    // Descriptors of stage 0 / weight buffer 0 at K step 0; every other one differs from them only in the start
    // address field (bits 0-13, address >> 4, which never carries: shared memory ends below 2^18), so the issue
    // loop adds small integers instead of rebuilding descriptors — the loop runs on one lane and its length is
    // what the tile rate sees.
    const uint64_t a_desc0 = make_sdesc(smem_u32(sStage), 16u, 1024u);
    const uint64_t b_desc0 = TRANS_W ? make_sdesc(smem_u32(sW), 16u, 1024u)
                                     : make_sdesc(smem_u32(sW), (uint32_t)p.k_dim * 128u, TF32 ? 512u : 1024u, TF32 ? 1u : 2u);
    const uint32_t b_kc_step = TRANS_W ? (uint32_t)p.n_dim * 8u : (uint32_t)EPR * 8u;  // one 128-byte K chunk further, in 16-byte units
    const uint32_t b_ks_step = TRANS_W ? 2u : (32u / ES) * 8u;                          // one 32-byte MMA step further
    G3Walk cur;
    cur.init(tile_start, n_seg, t0);
    int s = 0;
    uint32_t ph = 0;
    int cur_w = -1, n_load = -1, wb = 0, tile_i = 0;
    // One lane runs the whole loop — waits, issue, commits — so that no warp-wide hand-shake sits between a
    // stage landing and its MMAs; the other lanes wait at the end.
    if (lane == 0)
    for (int t = t0; t < t1 && ok; ++t, ++tile_i) {
      const int buf = tile_i & (cfg.n_tbuf - 1);
      const uint32_t use = (uint32_t)tile_i >> cfg.tbuf_shift;
      const int widx = g3_widx(cur, p);
      if (widx != cur_w) {  // same numbering of weight loads as in the producers
        ++n_load;
        wb = (cfg.n_wbuf == 2) ? (n_load & 1) : 0;
        cur_w = widx;
      }
      cur.next(tile_start, n_seg);
      const bool last_of_w = (t + 1 == t1) || g3_widx(cur, p) != cur_w;
      ok = mbar_wait(smem_u32(&sh->tmem_empty[buf]), (use & 1u) ^ 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)(buf * cfg.n_acc);
      const uint64_t b_desc_w = b_desc0 + (uint64_t)((uint32_t)wb * ((uint32_t)cfg.w_bytes >> 4));
      for (int kc = 0; kc < kch && ok; ++kc) {
        ok = mbar_wait(smem_u32(&sh->full[s]), ph, abort_flag);
        if (!ok) break;
        {
          fence_proxy_async();  // the stage was written through cp.async; the MMA reads it through the async proxy
          tc_fence_after();
          const uint64_t a_desc_s = a_desc0 + (uint64_t)((uint32_t)s * (G3_STAGE_BYTES >> 4));
          const uint64_t b_desc_kc = b_desc_w + (uint64_t)((uint32_t)kc * b_kc_step);
          const int n_ks = FULL ? 4 : min(4, (k_bytes - kc * 128) >> 5);  // 32-byte MMA steps this chunk holds
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            if (!FULL && ks >= n_ks) break;
            // A (K-major): 32 bytes further along the row per step.  B: MN-major (forward) steps 32 / ES rows of
            // 128 bytes, K-major (dgrad) 32 bytes along the row.
            mma_ss<TF32>(d_tmem, a_desc_s + (uint64_t)(ks * 2), b_desc_kc + (uint64_t)((uint32_t)ks * b_ks_step), idesc, (kc | ks) != 0);
          }
          mma_commit(smem_u32(&sh->empty[s]));
          if (kc == kch - 1) {
            mma_commit(smem_u32(&sh->tmem_full[buf]));
            if (last_of_w) mma_commit(smem_u32(&sh->w_free[wb]));
          }
        }
        if (++s == n_stage) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-7)
    // Two groups of four warps take alternate tiles, so that one group's TMEM reads and conversions run
    // while the other group's reds drain.  Warp q of a group owns TMEM lanes 32 q .. 32 q + 31 (a warp
    // may only read the lane quarter given by its index mod 4), i.e. tile rows 32 q .. 32 q + 31, and
    // walks the output row in 128-byte blocks: tcgen05.ld -> convert -> private patch -> reds.
    const int grp = warp >> 2, q4 = warp & 3;
    const uint32_t row_bytes = (uint32_t)p.n_dim * ES;
    constexpr uint32_t BLK_COLS = 128 / ES;  // accumulator columns per 128-byte block
    uint8_t* dst = static_cast<uint8_t*>(p.dst);
    uint8_t* patch = sPatch + warp * 4096;  // 32 rows x 128 bytes, private to the warp
    const uint32_t sw7 = (uint32_t)(lane & 7);
    // map entries of tile row 32 q + lane (-1 beyond the tile)
    const uint32_t ring = smem_u32(sRing) + (uint32_t)((G3_PROD_WARPS + 2 * warp) * G3_RING_SLOTS * 128 + lane * 4);
    auto fetch_entries = [&](const G3Walk& w, int slot) {  // gather entry -> ring[slot], scatter entry -> ring[SLOTS + slot]
      const G3Tile ti = g3_tile(w, p, kpos_s);
      const int row = 32 * q4 + lane;
      const uint32_t dg = ring + (uint32_t)slot * 128u, ds = dg + G3_RING_SLOTS * 128u;
      if (row < ti.cnt && !ti.dense) {
        cp_async4(dg, p.gather_map + ti.base + row);
        cp_async4(ds, p.scatter_map + ti.base + row);
      } else {
        const int v = row < ti.cnt ? ti.base + row : -1;
        st_shared_i32(dg, v);
        st_shared_i32(ds, v);
      }
    };
    if (t0 + grp < t1) {
      G3Walk pf;
      pf.init(tile_start, n_seg, t0 + grp);
      fetch_entries(pf, 0);
      cp_async_commit();
      pf.next(tile_start, n_seg);
      pf.next(tile_start, n_seg);
      if (pf.t < t1) fetch_entries(pf, 1);
      cp_async_commit();
      pf.next(tile_start, n_seg);
      pf.next(tile_start, n_seg);
      int own_i = 0;  // tiles of this group so far
      for (int t = t0 + grp; t < t1 && ok; t += 2) {
        const int tile_i = t - t0;
        if (pf.t < t1) fetch_entries(pf, (own_i + 2) & (G3_RING_SLOTS - 1));
        cp_async_commit();
        pf.next(tile_start, n_seg);
        pf.next(tile_start, n_seg);
        cp_async_wait<2>();  // this tile's entries (fetched two of the group's tiles ago) have landed
        const uint32_t slot = (uint32_t)(own_i & (G3_RING_SLOTS - 1));
        const int g0 = ld_shared_i32(ring + slot * 128u), s0 = ld_shared_i32(ring + (G3_RING_SLOTS + slot) * 128u);
        ++own_i;
        const int srow = pair_ok(g0, s0) ? s0 : -1;  // an entry outside the tensors: the pair is skipped
        const int buf = tile_i & (cfg.n_tbuf - 1);
        const uint32_t use = (uint32_t)tile_i >> cfg.tbuf_shift;
        ok = g3_wait(&sh->tmem_full[buf], use & 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(buf * cfg.n_acc);
        for (uint32_t cb = 0; cb < row_bytes; cb += 128) {
          // bytes of this block that belong to the row; `lpe` lanes share a row in the reds below
          const uint32_t vb = FULL ? 128u : min(128u, row_bytes - cb);
          const uint32_t lpe = (FULL || vb > 64) ? 8u : (vb > 32 ? 4u : 2u), rpe = 32u / lpe;
          const uint32_t ch = (uint32_t)lane % lpe, rsub = (uint32_t)lane / lpe;  // red: chunk ch of rows rsub + rpe u
          const uint32_t col0 = cb / ES;
          // 16 accumulator columns at a time: few registers in flight (a warp scheduler holding five warps of this
          // CTA leaves each thread about a hundred)
#pragma unroll
          for (uint32_t c0 = 0; c0 < BLK_COLS; c0 += 16) {
            uint32_t v[16];
            tmem_ld16(taddr + col0 + c0, v);
            tmem_ld_wait();
            if (TF32) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                *reinterpret_cast<uint4*>(patch + lane * 128 + (((uint32_t)(c0 / 4 + k) ^ sw7) << 4)) = make_uint4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
            } else {
              uint32_t h[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) h[k] = pack_half2(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
              *reinterpret_cast<uint4*>(patch + lane * 128 + (((c0 / 8) ^ sw7) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
              *reinterpret_cast<uint4*>(patch + lane * 128 + (((c0 / 8 + 1) ^ sw7) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
            }
          }
          if (cb + 128 >= row_bytes) {
            // accumulator fully read: hand the TMEM buffer back before the last reds go out
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->tmem_empty[buf]));
          }
          __syncwarp();
          uint8_t* dcol = dst + cb + (ch << 4);
          const bool ch_ok = FULL || (ch << 4) < vb;
#pragma unroll
          for (uint32_t u = 0; u < 8; ++u) {
            if (!FULL && u >= lpe) break;  // 32 rows = lpe passes of rpe rows
            const uint32_t r = rsub + rpe * u;
            const int sr = __shfl_sync(0xffffffffu, srow, r);
            const uint4 v = *reinterpret_cast<const uint4*>(patch + r * 128 + ((ch ^ (r & 7)) << 4));
            if (sr >= 0 && ch_ok) {
              uint8_t* o = dcol + (size_t)sr * row_bytes;
              if (TF32) red_add_v4(reinterpret_cast<float*>(o), __uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
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
  if (warp == G3_MMA_WARP) tmem_dealloc(tmem_base, tmem_cols);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// Shared-memory plan of a forward (trans = false) or dgrad (trans = true) launch.  Returns false when the
// shape is outside what the kernel takes or does not fit `max_smem`: the one place that decides it, used by
// the launcher and by the kernel-family query alike.
inline bool g3_plan(int c_in, int c_out, int es, int k_vol, int max_smem, bool trans, G3Config* cfg) {
  if (!umma_supported(c_in, c_out, es)) return false;
  const int k_dim = trans ? c_out : c_in, n_dim = trans ? c_in : c_out;
  const int epr = 128 / es;
  cfg->kch = (k_dim * es + 127) / 128;
  cfg->n_acc = (n_dim + epr - 1) / epr * epr;
  cfg->n_mma = trans ? n_dim : cfg->n_acc;
  cfg->w_bytes = trans ? n_dim * 128 * cfg->kch : k_dim * 128 * (cfg->n_acc / epr);
  cfg->n_tbuf = (4 * cfg->n_acc <= 512) ? 4 : 2;
  cfg->tbuf_shift = cfg->n_tbuf == 4 ? 2 : 1;
  const int table = ((2 * k_vol + 3) * 4 + 15) & ~15;
  const int fixed = 1024 + G3_PATCH_BYTES + G3_RING_BYTES + G3_SHARED_BYTES + table;
  // two weight buffers if at least four gather stages still fit beside them
  cfg->n_wbuf = (fixed + 2 * cfg->w_bytes + 4 * G3_STAGE_BYTES <= max_smem) ? 2 : 1;
  cfg->n_stage = (max_smem - fixed - cfg->n_wbuf * cfg->w_bytes) / G3_STAGE_BYTES;
  if (cfg->n_stage > G3_MAX_STAGES) cfg->n_stage = G3_MAX_STAGES;
  if (cfg->n_stage < 2) return false;
  cfg->smem = fixed + cfg->n_wbuf * cfg->w_bytes + cfg->n_stage * G3_STAGE_BYTES;
  return true;
}

// cudaFuncSetAttribute is needed once per kernel and device; `granted` remembers it (any thread may call)
template <typename K>
inline int ensure_smem(K kernel, int bytes, std::atomic<int>* granted /* [64], by device */) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (granted[dev].load(std::memory_order_acquire) >= bytes) return 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -1;
  granted[dev].store(bytes, std::memory_order_release);
  return 0;
}

template <bool TF32, bool TRANS_W, bool FULL>
inline int g3_launch_as(const GmsParams& p, const G3Config& cfg, cudaStream_t st, int sms, int max_smem) {
  static std::atomic<int> granted[64];
  if (int rc = ensure_smem(umma_gms3_kernel<TF32, TRANS_W, FULL>, max_smem, granted)) return rc;
  return launch_pdl(umma_gms3_kernel<TF32, TRANS_W, FULL>, sms, G3_THREADS, (size_t)cfg.smem, st, p, cfg) == cudaSuccess ? 0 : -1;
}
template <bool TF32, bool TRANS_W>
inline int g3_launch(const GmsParams& p, const G3Config& cfg, cudaStream_t st, int sms, int max_smem) {
  const int es = TF32 ? 4 : 2;
  const bool full = (p.c_in * es) % 128 == 0 && (p.c_out * es) % 128 == 0;
  return full ? g3_launch_as<TF32, TRANS_W, true>(p, cfg, st, sms, max_smem) : g3_launch_as<TF32, TRANS_W, false>(p, cfg, st, sms, max_smem);
}

// 0 launched, 1 the pointers are not 16-byte aligned or the shape has no plan (the caller takes the CUDA-core
// path and counts it), < 0 CUDA error
inline int launch_umma_gms3(const GmsParams& p, bool trans, bool f16, cudaStream_t st, int sms, int max_smem) {
  if ((reinterpret_cast<uintptr_t>(p.src) | reinterpret_cast<uintptr_t>(p.weights) | reinterpret_cast<uintptr_t>(p.dst)) & 15) return 1;
  G3Config cfg;
  if (!g3_plan(p.c_in, p.c_out, f16 ? 2 : 4, p.k_vol, max_smem, trans, &cfg)) return 1;
  if (f16) return trans ? g3_launch<false, true>(p, cfg, st, sms, max_smem) : g3_launch<false, false>(p, cfg, st, sms, max_smem);
  return trans ? g3_launch<true, true>(p, cfg, st, sms, max_smem) : g3_launch<true, false>(p, cfg, st, sms, max_smem);
}

}  // namespace fgms
