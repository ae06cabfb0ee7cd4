// Weight gradient on tcgen05, warp-specialised with private hand-offs only.
//
//   dw[k] (c_in x c_out, fp32) += sum over the pairs j of offset k of feats[in_map[j]]^T (x) out_grad[out_map[j]]
//
// The pair index is the contraction index: both operands are gathered rows used MN-major.
//   A = feats rows     [pb pairs x c_in ]   M = c_in  (tiles of 128 rows; the last tile has 64 when at most 64 rows remain)
//   B = out_grad rows  [pb pairs x c_out]   N = c_out rounded up to a whole 128-byte piece
// Rows are staged in 128-byte pieces.  A piece that a short row fills only in part, or that exists only to
// complete the last row tile, holds stale shared memory beyond the row: those values reach accumulator rows
// >= c_in and columns >= c_out only, which are never written out.
// One persistent CTA per SM walks a contiguous range of pb-pair stages.  The accumulator stays in TMEM
// while consecutive stages belong to the same offset and is flushed with 16-byte vector reds to the
// fp32 gradient when the offset changes (split-K across CTAs).
//
//   producers (8 warps)  warp w owns rows [w pb/8, (w+1) pb/8) of every stage: it fetches those rows' map
//                        entries from global memory four stages ahead and gathers both operands with
//                        16-byte cp.async;
//   MMA warp             one lane issues tcgen05.mma per stage and commits the stage back to the producers;
//                        on a change of offset it commits the accumulator to the epilogue;
//   epilogue (4 warps)   tcgen05.ld -> private 4 KB patch -> reds with consecutive lanes on consecutive
//                        addresses of one gradient row.
// All waits are bounded; a wait that runs out sets the CTA's abort flag and every role leaves its loop.
#pragma once
#include "common.cuh"
#include "umma.cuh"
#include "umma_gms3.cuh"  // G3Walk, g3_wait

namespace fgms {

constexpr int W3_EPI_WARPS = 4;
constexpr int W3_MMA_WARP = 4;
constexpr int W3_PROD_WARP0 = 5;
constexpr int W3_PROD_WARPS = 8;
constexpr int W3_PROD_THREADS = W3_PROD_WARPS * 32;
constexpr int W3_THREADS = (W3_PROD_WARP0 + W3_PROD_WARPS) * 32;
__device__ __forceinline__ int w3_producer_index(int warp) { return warp - W3_PROD_WARP0; }  // < 0: no producer
constexpr int W3_MAX_STAGES = 12;
constexpr int W3_MAX_PB = 256;
constexpr int W3_PATCH_BYTES = W3_EPI_WARPS * 4096;
constexpr int W3_PREFETCH = 4;  // map entries are fetched this many stages ahead

struct W3Shared {
  uint64_t full[W3_MAX_STAGES];
  uint64_t empty[W3_MAX_STAGES];  // used at the first stage of every group: the group's stages have been consumed
  uint64_t tmem_full[4];
  uint64_t tmem_empty[4];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int W3_SHARED_BYTES = (sizeof(W3Shared) + 15) & ~15;

struct W3Config {
  int pb;         // pairs per stage: 32, 64, 128 or 256
  int pack;       // pairs that share one staged row (their rows side by side): 1, 2 or 4
  int slot_a, slot_b;  // packed stages: bytes a pair's row takes in the staged row of A / of B
  int n_mtile;    // 1 or 2 accumulator row tiles: all of 128 rows but possibly the last
  int last_m;     // rows of the last tile's MMA: 128, or 64 when at most 64 rows remain
  int alias;      // 1: the last tile's second piece is its first one read again (descriptor LBO = 0) instead of a
                  //    piece of its own — tf32 with at most 32 rows left: an M = 64 MMA reads two 32-row pieces, only
                  //    one is real, and the rows it repeats land in accumulator rows that are never written out
  int pa, pbp;    // 128-byte pieces per staged row of A (enough for every row tile) and of B (n_acc columns)
  int n_acc;      // TMEM columns of one row tile: c_out rounded up to a whole piece
  int smem;       // dynamic shared memory of the launch
  int n_buf;      // TMEM accumulator sets: 1, 2 or 4
  int buf_shift;  // log2(n_buf)
  int n_stage;    // a multiple of `group`
  int group;      // stages handed back to the producers by one tcgen05.commit (a commit drains the MMA pipe)
};

// stage t of the table: first pair and number of pairs
__device__ __forceinline__ void w3_stage(const G3Walk& w, int pb, const int* kpos_s, int* base, int* cnt) {
  const int lt = w.t - w.seg_first;
  const int seg_base = kpos_s[w.seg];
  *base = seg_base + lt * pb;
  *cnt = min(pb, kpos_s[w.seg + 1] - seg_base - lt * pb);
}

// FULL: both row lengths are whole 128-byte pieces; the producers' copy loops then carry no per-chunk test.
// PACKED: several pairs share a staged row (cfg.pack > 1); the unpacked instantiations carry none of its arithmetic.
template <bool TF32, bool FULL, bool PACKED>
__global__ void __launch_bounds__(W3_THREADS, 1) umma_wgrad3_kernel(WgradParams p, W3Config cfg) {
  using namespace umma;
  constexpr int ES = TF32 ? 4 : 2;
  constexpr int UK = 32 / ES;  // contraction length of one MMA
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int pb = cfg.pb, n_stage = cfg.n_stage;
  const int kr = PACKED ? pb / cfg.pack : pb;  // staged rows (contraction steps) per stage
  const uint32_t a_bytes = (uint32_t)kr * 128u * cfg.pa;
  const uint32_t stage_bytes = (uint32_t)kr * 128u * (cfg.pa + cfg.pbp);
  uint8_t* sStage = smem;
  uint8_t* sPatch = sStage + (size_t)n_stage * stage_bytes;
  W3Shared* sh = reinterpret_cast<W3Shared*>(sPatch + W3_PATCH_BYTES);
  int* tile_start = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(sh) + W3_SHARED_BYTES);  // [k_vol + 2]
  int* kpos_s = tile_start + p.k_vol + 2;                                                        // [k_vol + 1]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_seg = p.k_vol + 1;
  volatile int* abort_flag = &sh->abort_flag;
  const uint32_t lbo = (uint32_t)kr * 128u;  // next 128 bytes of every staged row
  const uint32_t buf_cols = (uint32_t)(cfg.n_mtile * cfg.n_acc);

  if (tid == 0) {
    for (int s = 0; s < n_stage; ++s) {
      mbar_init(smem_u32(&sh->full[s]), W3_PROD_THREADS);  // one hardware arrival per producer thread
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(smem_u32(&sh->tmem_full[b]), 1);
      mbar_init(smem_u32(&sh->tmem_empty[b]), W3_EPI_WARPS);
    }
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  // TMEM allocation overlaps the first global loads below
  uint32_t tmem_cols = 32;
  while (tmem_cols < buf_cols * (uint32_t)cfg.n_buf) tmem_cols <<= 1;
  if (warp == W3_MMA_WARP) {
    tmem_alloc(smem_u32(&sh->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  // everything above touches no global memory; from here on the previous kernel's results may be needed
  griddep_wait();
  griddep_launch_dependents();
  build_tile_table(pb, p.kpos, p.pairs, p.k_vol, 0, kpos_s, tile_start);  // syncs the CTA
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);
  bool ok = true;

  if (t0 >= t1) {
    // nothing for this CTA
  } else if (w3_producer_index(warp) >= 0) {
    // ------------------------------------------------------------------ producers
    const int pw = w3_producer_index(warp);
    const int rpw = pb / W3_PROD_WARPS;  // rows of a stage owned by this warp: 4, 8, 16 or 32
    const uint8_t* feats = static_cast<const uint8_t*>(p.feats);
    const uint8_t* og = static_cast<const uint8_t*>(p.out_grad);
    const uint32_t a_row_bytes = (uint32_t)p.c_in * ES, b_row_bytes = (uint32_t)p.c_out * ES;
    // `lpr` lanes share a row, one 16-byte chunk each: 8 when the longer of the two rows exceeds 64 bytes, 4 / 2
    // for rows of at most 64 / 32 bytes, so that a warp-wide copy of short rows still carries 32 chunks (8 / 16
    // rows instead of 4).  The time of a stage's copies goes with the number of warp-wide copy rounds, not with
    // the bytes they carry.
    const uint32_t max_row = a_row_bytes > b_row_bytes ? a_row_bytes : b_row_bytes;
    int lpr = (FULL || max_row > 64) ? 8 : (max_row > 32 ? 4 : 2);
    if (32 / lpr > rpw) lpr = 8;         // fewer rows per warp than such a round would cover
    const int rpp = 32 / lpr;            // rows per round: 4, 8 or 16
    const int n_pass = rpw / rpp;        // rounds per stage: 1 .. 8
    // Lane (rs, c) = (lane / lpr, lane % lpr) copies 16-byte chunk c of every 128-byte piece of the rows
    // rs, rs + rpp, ... of the warp's block: one shuffle and one address per row, then one cp.async per
    // piece at a fixed distance (128 bytes in global memory, `lbo` in shared memory).
    const int rs = lane / lpr, cc = lane % lpr;
    // 128-byte pieces of a row this lane's 16-byte chunk exists in (the last piece of a row that is no whole
    // number of pieces is filled in part): 0 .. 8
    const int nha = FULL ? (int)a_row_bytes / 128 : ((int)a_row_bytes - cc * 16 + 127) / 128;
    const int nhb = FULL ? (int)b_row_bytes / 128 : ((int)b_row_bytes - cc * 16 + 127) / 128;
    // piece 0 of row rs + rpp u, relative to the operand's start in the stage: rows 8 apart are 1024 bytes apart in
    // both layouts, so with 4 rows per round two offsets (u even / odd) and a multiple of 1024 give all of them,
    // with 8 or 16 rows per round one offset and a multiple of 1024 or 2048
    uint32_t dst_rel[2];
    const int pack = PACKED ? cfg.pack : 1;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint32_t row = (uint32_t)(pw * rpw + rs + 4 * u);
      dst_rel[u] = TF32 ? mnmajor32_offset(row, (uint32_t)cc * 16u, lbo, 512u) : mnmajor_offset(row, (uint32_t)cc * 16u, lbo, 1024u);
    }
    const bool four = rpp == 4;
    const uint32_t u_step = four ? 1024u : (uint32_t)(rpp >> 3) * 1024u;
    // Packed stages: pair j of the stage sits in staged row j / pack, its rows at byte (j % pack) * slot_a of A and
    // (j % pack) * slot_b of B (a position beyond 128 bytes is a further piece).  Round u covers the staged row
    // row0 + u * rpp / pack; the offsets are worked out per round.
    const uint32_t pk_row0 = (uint32_t)(pw * rpw + rs) / (uint32_t)pack, pk_step = (uint32_t)(rpp / pack);
    const uint32_t pk_byte_a = (uint32_t)((pw * rpw + rs) % pack) * (uint32_t)cfg.slot_a + (uint32_t)cc * 16u;
    const uint32_t pk_byte_b = (uint32_t)((pw * rpw + rs) % pack) * (uint32_t)cfg.slot_b + (uint32_t)cc * 16u;
    const uint8_t* feats_c = feats + cc * 16;
    const uint8_t* og_c = og + cc * 16;
    // lane r < rpw fetches both map entries of the warp's row r (-1 beyond the stage)
    auto load_entry = [&](const G3Walk& w, int* ea, int* eb) {
      int base, cnt;
      w3_stage(w, pb, kpos_s, &base, &cnt);
      const int row = pw * rpw + lane;
      *ea = *eb = -1;
      if (lane < rpw && row < cnt) {
        *ea = __ldg(p.in_map + base + row);
        *eb = __ldg(p.out_map + base + row);
      }
    };
    G3Walk pf;
    pf.init(tile_start, n_seg, t0);
    int ea[W3_PREFETCH], eb[W3_PREFETCH];
#pragma unroll
    for (int d = 0; d < W3_PREFETCH; ++d) {
      ea[d] = eb[d] = -1;
      if (pf.t < t1) load_entry(pf, &ea[d], &eb[d]);
      pf.next(tile_start, n_seg);
    }
    int s = 0, sg = 0;  // stage, and its position in its group
    uint32_t ph = 0;
    for (int t = t0; t < t1 && ok; ++t) {
      int cur_a = ea[0], cur_b = eb[0];
#pragma unroll
      for (int d = 0; d + 1 < W3_PREFETCH; ++d) { ea[d] = ea[d + 1]; eb[d] = eb[d + 1]; }
      ea[W3_PREFETCH - 1] = eb[W3_PREFETCH - 1] = -1;
      if (pf.t < t1) load_entry(pf, &ea[W3_PREFETCH - 1], &eb[W3_PREFETCH - 1]);
      pf.next(tile_start, n_seg);
      // a pair is used only if both its entries are inside the tensors
      if (!((unsigned)cur_a < (unsigned)p.n_in && (unsigned)cur_b < (unsigned)p.n_out)) {
        if (cur_a != -1 || cur_b != -1) report_problem();  // counted once per skipped pair
        cur_a = cur_b = -1;
      }
      if (sg == 0) {
        ok = g3_wait(&sh->empty[s], ph ^ 1u, abort_flag);
        if (!ok) break;
      }
      const uint32_t sa = smem_u32(sStage + (size_t)s * stage_bytes);
      const uint32_t sb = sa + a_bytes;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (u < n_pass) {
          const int ia = __shfl_sync(0xffffffffu, cur_a, rs + rpp * u);
          const int ib = __shfl_sync(0xffffffffu, cur_b, rs + rpp * u);
          const uint32_t na = ia >= 0 ? 16u : 0u, nb = ib >= 0 ? 16u : 0u;  // 0 bytes read: the chunk is zero-filled
          const uint8_t* pa = feats_c + (size_t)max(ia, 0) * a_row_bytes;
          const uint8_t* pb_ = og_c + (size_t)max(ib, 0) * b_row_bytes;
          uint32_t rel_a, rel_b;
          if (!PACKED) {
            rel_a = rel_b = four ? dst_rel[u & 1] + (uint32_t)(u >> 1) * 1024u : dst_rel[0] + (uint32_t)u * u_step;
          } else {
            const uint32_t row = pk_row0 + (uint32_t)u * pk_step;
            rel_a = TF32 ? mnmajor32_offset(row, pk_byte_a, lbo, 512u) : mnmajor_offset(row, pk_byte_a, lbo, 1024u);
            rel_b = TF32 ? mnmajor32_offset(row, pk_byte_b, lbo, 512u) : mnmajor_offset(row, pk_byte_b, lbo, 1024u);
          }
          const uint32_t da = sa + rel_a, db = sb + rel_b;
#pragma unroll
          for (int h = 0; h < 8; ++h)
            if (h < nha) cp_async16_n(da + (uint32_t)h * lbo, pa + h * 128, na);
#pragma unroll
          for (int h = 0; h < 8; ++h)
            if (h < nhb) cp_async16_n(db + (uint32_t)h * lbo, pb_ + h * 128, nb);
        }
      }
      // the stage's barrier hears from this thread when everything it has issued so far has landed
      cp_async_arrive_noinc(smem_u32(&sh->full[s]));
      if (++sg == cfg.group) sg = 0;
      if (++s == n_stage) { s = 0; ph ^= 1u; }
    }
  } else if (warp == W3_MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc_full = make_idesc(TF32, true, true, 128, cfg.n_acc);
    const uint32_t idesc_last = make_idesc(TF32, true, true, cfg.last_m, cfg.n_acc);
    const uint32_t sbo = TF32 ? 512u : 1024u, ltype = TF32 ? 1u : 2u;
    const uint32_t mtile_stride = (uint32_t)ES * lbo;  // a 128-row tile spans 128 * ES / 128 pieces
    const uint32_t last_lbo = cfg.alias ? 0u : lbo;
    // Descriptors of stage 0 at K step 0 (A: one per row tile); all others differ only in the start-address field
    // (address >> 4, no carry out of it), so the issue loop adds small integers instead of rebuilding them
    const uint32_t stage0 = smem_u32(sStage);
    const uint64_t b_desc0 = make_sdesc(stage0 + a_bytes, lbo, sbo, ltype);
    uint64_t a_desc0[2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
      a_desc0[mt] = make_sdesc(stage0 + (uint32_t)mt * mtile_stride, mt + 1 == cfg.n_mtile ? last_lbo : lbo, sbo, ltype);
    const uint32_t ks_step = (uint32_t)UK * 8u;  // UK contraction rows of 128 bytes, in 16-byte units
    G3Walk cur;
    cur.init(tile_start, n_seg, t0);
    int s = 0, sg = 0, run_i = 0, cur_seg = -1;
    uint32_t ph = 0;
    bool first = true;
    // One lane runs the whole loop — waits, issue, commits — so that no warp-wide hand-shake sits between a
    // stage landing and its MMAs; the other lanes wait at the end.
    if (lane == 0) {
    for (int t = t0; t < t1 && ok; ++t) {
      if (cur.seg != cur_seg) {
        if (cur_seg >= 0) {
          mma_commit(smem_u32(&sh->tmem_full[run_i & (cfg.n_buf - 1)]));
          ++run_i;
        }
        cur_seg = cur.seg;
        first = true;
        const uint32_t use = (uint32_t)run_i >> cfg.buf_shift;
        ok = mbar_wait(smem_u32(&sh->tmem_empty[run_i & (cfg.n_buf - 1)]), (use & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
      }
      const int buf = run_i & (cfg.n_buf - 1);
      ok = mbar_wait(smem_u32(&sh->full[s]), ph, abort_flag);
      if (!ok) break;
      {
        fence_proxy_async();  // the stage was written through cp.async; the MMA reads it through the async proxy
        tc_fence_after();
        const uint64_t s_off = (uint64_t)((uint32_t)s * (stage_bytes >> 4));
        const uint32_t d0 = tmem_base + (uint32_t)buf * buf_cols;
        for (int ks = 0; ks < kr / UK; ++ks) {
          const uint64_t off = s_off + (uint64_t)((uint32_t)ks * ks_step);
          mma_ss<TF32>(d0, a_desc0[0] + off, b_desc0 + off, cfg.n_mtile == 1 ? idesc_last : idesc_full, !(first && ks == 0));
          if (cfg.n_mtile == 2)
            mma_ss<TF32>(d0 + (uint32_t)cfg.n_acc, a_desc0[1] + off, b_desc0 + off, idesc_last, !(first && ks == 0));
        }
        // one commit per group of stages (and one for the CTA's last stage, which nobody waits for)
        if (sg == cfg.group - 1 || t + 1 == t1) mma_commit(smem_u32(&sh->empty[s - sg]));
      }
      first = false;
      if (++sg == cfg.group) sg = 0;
      if (++s == n_stage) { s = 0; ph ^= 1u; }
      cur.next(tile_start, n_seg);
    }
    if (ok && cur_seg >= 0) mma_commit(smem_u32(&sh->tmem_full[run_i & (cfg.n_buf - 1)]));
    }
    __syncwarp();
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  } else if (warp < W3_EPI_WARPS) {
    // ------------------------------------------------------------------ epilogue (warps 0-3)
    // Thread (warp, lane) holds accumulator row m in its TMEM lane.  32 columns of the warp's 32 rows
    // go through the warp's patch so that eight consecutive lanes add 128 consecutive bytes of one row.
    uint8_t* patch = sPatch + warp * 4096;
    const uint32_t sw7 = (uint32_t)(lane & 7);
    const uint32_t ch = (uint32_t)(lane & 7), rsub = (uint32_t)(lane >> 3);
    // Packed stages: staged row k holds `pack` pairs side by side, in A and in B, so the accumulator is pack x pack
    // blocks of slot_m x slot_n elements of which the diagonal ones are sums over pairs (block (s, s): the pairs in
    // position s) and the others mix two pairs' rows and are dropped.  A warp's rows (32 of a 128-row accumulator,
    // 16 of a 64-row one) lie in one block row; it adds columns [col_base, col_base + c_out) of its rows to gradient
    // rows (row - row_base).  (tf32 with at most 32 staged elements: the 64-row MMA reads them twice, rows 32 .. 63
    // repeat rows 0 .. 31 and are dropped.)
    const int slot_m = PACKED ? cfg.slot_a / ES : 0, slot_n = PACKED ? cfg.slot_b / ES : 0;
    const int warp_row0 = (cfg.last_m == 128 ? 32 : 16) * warp;  // packed stages have one row tile
    const bool blk_ok = !PACKED || warp_row0 < cfg.pack * slot_m;
    const int blk = (PACKED && blk_ok) ? warp_row0 / slot_m : 0;
    const int row_base = blk * slot_m, col_base = blk * slot_n;
    int run_i = 0;
    int t = t0;
    while (t < t1 && ok) {
      const int seg = find_segment(tile_start, n_seg, t);
      t = min(t1, tile_start[seg + 1]);  // this CTA's stages of the offset end here
      const int buf = run_i & (cfg.n_buf - 1);
      const uint32_t use = (uint32_t)run_i >> cfg.buf_shift;
      ok = g3_wait(&sh->tmem_full[buf], use & 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      float* dwk = p.dw + (size_t)seg * p.c_in * p.c_out;
      if (!TF32 && p.dw_f16 != nullptr) {
        // fp16 destination: 64 columns (128 bytes of fp16) of the warp's 32 rows per round
        __half* dwk16 = p.dw_f16 + (size_t)seg * p.c_in * p.c_out;
        for (int mt = 0; mt < cfg.n_mtile; ++mt) {
          const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)buf * buf_cols + (uint32_t)(mt * cfg.n_acc);
          const bool m128 = mt + 1 < cfg.n_mtile || cfg.last_m == 128;
          for (int c0 = 0; c0 < p.c_out; c0 += 64) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {  // 16 columns at a time: few registers in flight
              uint32_t v[16], h[8];
              if (PACKED && c0 + 16 * q >= slot_n) break;  // the block's columns end here
              tmem_ld16(taddr + col_base + c0 + 16 * q, v);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 8; ++k) h[k] = pack_half2(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
              *reinterpret_cast<uint4*>(patch + lane * 128 + (((uint32_t)(2 * q) ^ sw7) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
              *reinterpret_cast<uint4*>(patch + lane * 128 + (((uint32_t)(2 * q + 1) ^ sw7) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
            }
            __syncwarp();
#pragma unroll
            for (uint32_t u = 0; u < 8; ++u) {
              const uint32_t r = rsub + 4 * u;
              int m;
              if (m128) m = blk_ok ? mt * 128 + warp * 32 + (int)r - row_base : -1;
              else m = (r < 16 && blk_ok) ? mt * 128 + warp * 16 + (int)r - row_base : -1;
              const uint4 v = *reinterpret_cast<const uint4*>(patch + r * 128 + ((ch ^ (r & 7)) << 4));
              if (m >= 0 && m < p.c_in && c0 + (int)(ch << 3) < p.c_out) red_add_h8(dwk16 + (size_t)m * p.c_out + c0 + (ch << 3), v.x, v.y, v.z, v.w);
            }
            __syncwarp();
          }
        }
      } else
      for (int mt = 0; mt < cfg.n_mtile; ++mt) {
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)buf * buf_cols + (uint32_t)(mt * cfg.n_acc);
        const bool m128 = mt + 1 < cfg.n_mtile || cfg.last_m == 128;
        for (int c0 = 0; c0 < p.c_out; c0 += 32) {
          uint32_t v0[16], v1[16];
          tmem_ld16(taddr + col_base + c0, v0);
          if (!PACKED || slot_n - c0 > 16) {
            tmem_ld16(taddr + col_base + c0 + 16, v1);
          } else {  // the block has 16 columns: the next ones belong to another block (or to no accumulator at all)
#pragma unroll
            for (int k = 0; k < 16; ++k) v1[k] = 0u;
          }
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            *reinterpret_cast<uint4*>(patch + lane * 128 + (((uint32_t)k ^ sw7) << 4)) = make_uint4(v0[4 * k], v0[4 * k + 1], v0[4 * k + 2], v0[4 * k + 3]);
            *reinterpret_cast<uint4*>(patch + lane * 128 + (((uint32_t)(4 + k) ^ sw7) << 4)) = make_uint4(v1[4 * k], v1[4 * k + 1], v1[4 * k + 2], v1[4 * k + 3]);
          }
          __syncwarp();
#pragma unroll
          for (uint32_t u = 0; u < 8; ++u) {
            const uint32_t r = rsub + 4 * u;  // TMEM lane (within the warp's quarter) whose row this is
            // M = 128: lane r of warp w is row 32 w + r; M = 64: row i lives in lane (i / 16) * 32 + i % 16
            int m;
            if (m128) m = blk_ok ? mt * 128 + warp * 32 + (int)r - row_base : -1;
            else m = (r < 16 && blk_ok) ? mt * 128 + warp * 16 + (int)r - row_base : -1;
            const uint4 v = *reinterpret_cast<const uint4*>(patch + r * 128 + ((ch ^ (r & 7)) << 4));
            if (m >= 0 && m < p.c_in && c0 + (int)(ch << 2) < p.c_out)
              red_add_v4(dwk + (size_t)m * p.c_out + c0 + (ch << 2), __uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->tmem_empty[buf]));
      ++run_i;
    }
  }

  if (!ok && lane == 0) report_problem();
  cp_async_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == W3_MMA_WARP) tmem_dealloc(tmem_base, tmem_cols);
}

// Plan of a launch: accumulator row tiling for c_in, pieces per staged row, stage size and count.  Returns
// false for shapes the kernel does not take or that do not fit `max_smem`; used by the launcher and by the
// kernel-family query alike.
inline bool w3_plan(int c_in, int c_out, int es, int k_vol, int max_smem, W3Config* cfg) {
  if (!umma_supported(c_in, c_out, es)) return false;
  const int epr = 128 / es;  // elements per 128-byte piece
  // Packed stages: `pack` pairs share a staged row, their rows side by side in A and in B, so one MMA contracts
  // pack times as many pairs — an MMA of 64 x 64 x 16 costs what one of 128 x 128 x 16 does, and with rows of up to
  // 128 bytes the issue loop is what bounds the kernel.  The accumulator then holds pack x pack blocks; the epilogue
  // keeps the diagonal.  Rows of at most 32 / 64 bytes: 4 pairs in slots of 32 / 64 bytes (a 64 x 64 accumulator,
  // or 128 x 128 for the 64-byte slots of fp16: one MMA per 64 pairs).  Longer rows whose
  // lengths are powers of two: 2 pairs, each row its own slot, while both fit one 128-row, 256-column accumulator
  // (twice, so that two accumulators alternate) and three packed stages of 128 pairs fit shared memory — else the
  // shape is planned unpacked (second pass of the loop).
  const int a_row = c_in * es, b_row = c_out * es, max_row = a_row > b_row ? a_row : b_row;
  const bool pow2 = (a_row & (a_row - 1)) == 0 && (b_row & (b_row - 1)) == 0;
  for (int attempt = 0; attempt < 2; ++attempt) {
  cfg->pack = 1; cfg->slot_a = cfg->slot_b = 0;
  if (attempt == 0) {
    if (max_row <= 32) { cfg->pack = 4; cfg->slot_a = cfg->slot_b = 32; }
    else if (max_row <= 64) { cfg->pack = 4; cfg->slot_a = cfg->slot_b = 64; }
    else if (pow2 && 2 * c_in <= 128 && 2 * c_out <= 256) { cfg->pack = 2; cfg->slot_a = a_row; cfg->slot_b = b_row; }
    else continue;
  }
  // rows and columns of the accumulator
  const int m_eff = cfg->pack > 1 ? cfg->pack * cfg->slot_a / es : c_in;
  const int n_eff = cfg->pack > 1 ? cfg->pack * cfg->slot_b / es : c_out;
  cfg->n_mtile = (m_eff + 127) / 128;
  const int rem = m_eff - 128 * (cfg->n_mtile - 1);
  cfg->last_m = rem <= 64 ? 64 : 128;
  cfg->alias = (es == 4 && rem <= 32) ? 1 : 0;
  cfg->pa = (cfg->n_mtile - 1) * es + (cfg->last_m == 128 ? es : es / 2) - cfg->alias;  // a 128-row tile reads 128 / epr = es pieces
  cfg->n_acc = (n_eff + epr - 1) / epr * epr;
  cfg->pbp = cfg->n_acc / epr;
  const int buf_cols = cfg->n_mtile * cfg->n_acc;
  if (buf_cols > 512) { if (cfg->pack > 1) continue; return false; }
  cfg->n_buf = 4 * buf_cols <= 512 ? 4 : (2 * buf_cols <= 512 ? 2 : 1);
  cfg->buf_shift = cfg->n_buf == 4 ? 2 : (cfg->n_buf == 2 ? 1 : 0);
  // pairs per stage: 4, 8, 16 or 32 rows per producer warp (packed stages: always 32, the stage is small)
  int pb = W3_MAX_PB;
  const int fixed = 1024 + W3_PATCH_BYTES + W3_SHARED_BYTES + (((2 * k_vol + 3) * 4 + 15) & ~15);
  const int row_bytes = 128 * (cfg->pa + cfg->pbp) / cfg->pack;  // staged bytes per pair
  // keep at least three stages in flight; a packed stage keeps the producers' round a whole number of staged rows
  while (pb > (cfg->pack > 1 ? 128 : 32) && (max_smem - fixed) / (pb * row_bytes) < 3) pb >>= 1;
  int n_stage = (max_smem - fixed) / (pb * row_bytes);
  if (n_stage > W3_MAX_STAGES) n_stage = W3_MAX_STAGES;
  if (cfg->pack > 1 && n_stage < 3) continue;  // too large packed: plan it unpacked
  if (n_stage < 2) return false;
  // stages per commit: as many as leave three groups in flight
  cfg->group = 1;
  for (int g = 4; g >= 2; --g)
    if ((n_stage - n_stage % g) / g >= 3) { cfg->group = g; n_stage -= n_stage % g; break; }
  cfg->pb = pb;
  cfg->n_stage = n_stage;
  cfg->smem = fixed + n_stage * pb * row_bytes;
  return true;
  }
  return false;
}

template <bool TF32, bool FULL, bool PACKED>
inline int w3_launch_as(const WgradParams& p, const W3Config& cfg, cudaStream_t st, int sms, int max_smem) {
  static std::atomic<int> granted[64];
  if (int rc = ensure_smem(umma_wgrad3_kernel<TF32, FULL, PACKED>, max_smem, granted)) return rc;
  return launch_pdl(umma_wgrad3_kernel<TF32, FULL, PACKED>, sms, W3_THREADS, (size_t)cfg.smem, st, p, cfg) == cudaSuccess ? 0 : -1;
}
template <bool TF32>
inline int w3_launch(const WgradParams& p, const W3Config& cfg, cudaStream_t st, int sms, int max_smem) {
  const int es = TF32 ? 4 : 2;
  const bool full = (p.c_in * es) % 128 == 0 && (p.c_out * es) % 128 == 0;
  if (cfg.pack > 1)
    return full ? w3_launch_as<TF32, true, true>(p, cfg, st, sms, max_smem) : w3_launch_as<TF32, false, true>(p, cfg, st, sms, max_smem);
  return full ? w3_launch_as<TF32, true, false>(p, cfg, st, sms, max_smem) : w3_launch_as<TF32, false, false>(p, cfg, st, sms, max_smem);
}

// 0 launched, 1 the pointers are not 16-byte aligned or the shape has no plan (the caller takes the CUDA-core
// path and counts it), < 0 CUDA error
inline int launch_umma_wgrad3(const WgradParams& p, bool f16, cudaStream_t st, int sms, int max_smem) {
  if ((reinterpret_cast<uintptr_t>(p.feats) | reinterpret_cast<uintptr_t>(p.out_grad) | reinterpret_cast<uintptr_t>(p.dw) | reinterpret_cast<uintptr_t>(p.dw_f16)) & 15) return 1;
  W3Config cfg;
  if (!w3_plan(p.c_in, p.c_out, f16 ? 2 : 4, p.k_vol, max_smem, &cfg)) return 1;
  return f16 ? w3_launch<false>(p, cfg, st, sms, max_smem) : w3_launch<true>(p, cfg, st, sms, max_smem);
}

}  // namespace fgms
