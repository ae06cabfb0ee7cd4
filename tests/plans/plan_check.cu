// Host-side check of the launch plans of the tensor-core kernels (g3_plan, w3_plan) over every channel pair the
// kernels take: shared memory within the limit, enough stages, accumulators within the 512 TMEM columns, and the
// packing rules of the weight-gradient kernel.  Prints one line per violation; exit status = their number.
#include <cstdio>
#include "../../fgms_b200/csrc/umma_gms3.cuh"
#include "../../fgms_b200/csrc/umma_wgrad3.cuh"
using namespace fgms;

int main() {
  const int max_smem = 232448;  // B200: 227 KB per CTA
  int bad = 0, seen = 0, packed = 0;
  auto fail = [&](const char* what, int es, int ci, int co, int kv) {
    std::printf("%s: es %d, %d -> %d, k_vol %d\n", what, es, ci, co, kv);
    ++bad;
  };
  for (int es : {2, 4})
    for (int ci = 16; ci <= 256; ci += 16)
      for (int co = 16; co <= 256; co += 16)
        for (int kv : {1, 8, 27, 125}) {
          if (!umma_supported(ci, co, es)) { fail("multiple of 16 not supported", es, ci, co, kv); continue; }
          ++seen;
          for (int trans = 0; trans < 2; ++trans) {
            G3Config g;
            if (!g3_plan(ci, co, es, kv, max_smem, trans != 0, &g)) {
              // the one shape family without a plan: a weight operand that leaves no room for two stages
              const int k = trans ? co : ci, n = trans ? ci : co;
              if ((long long)k * n * es < 131072) fail("g3_plan refused a shape that should fit", es, ci, co, kv);
              continue;
            }
            if (g.smem > max_smem) fail("g3 smem over the limit", es, ci, co, kv);
            if (g.n_stage < 2 || g.n_stage > G3_MAX_STAGES) fail("g3 stage count", es, ci, co, kv);
            if (g.n_tbuf * g.n_acc > 512 || (g.n_tbuf != 2 && g.n_tbuf != 4)) fail("g3 accumulators", es, ci, co, kv);
            if (g.kch != ((trans ? co : ci) * es + 127) / 128) fail("g3 K chunks", es, ci, co, kv);
            if (g.n_acc < (trans ? ci : co) || g.n_acc % (128 / es)) fail("g3 accumulator width", es, ci, co, kv);
          }
          W3Config w;
          if (!w3_plan(ci, co, es, kv, max_smem, &w)) { fail("w3_plan refused", es, ci, co, kv); continue; }
          if (w.smem > max_smem) fail("w3 smem over the limit", es, ci, co, kv);
          if (w.n_stage < 3 && w.pb > 32) fail("w3 fewer than three stages", es, ci, co, kv);
          if (w.n_stage % w.group) fail("w3 stages no multiple of the group", es, ci, co, kv);
          if (w.n_buf * w.n_mtile * w.n_acc > 512) fail("w3 accumulators", es, ci, co, kv);
          if (w.pb % W3_PROD_WARPS || w.pb / W3_PROD_WARPS < 4 || w.pb > W3_MAX_PB) fail("w3 pairs per stage", es, ci, co, kv);
          if (w.pack > 1) {
            ++packed;
            const int m = w.pack * w.slot_a / es, n = w.pack * w.slot_b / es;
            if (w.slot_a < ci * es || w.slot_b < co * es) fail("w3 slot shorter than the row", es, ci, co, kv);
            if (w.n_mtile != 1 || m > 128 || n > 256 || n > w.n_acc) fail("w3 packed accumulator", es, ci, co, kv);
            if ((w.pb / W3_PROD_WARPS) % w.pack) fail("w3 a warp's rows no multiple of the pack", es, ci, co, kv);
            if (w.pa * 128 < (w.last_m == 128 ? 128 : 64) * es - (w.alias ? 128 : 0)) fail("w3 packed A pieces", es, ci, co, kv);
            if (w.n_buf < 2) fail("w3 packed stages with one accumulator", es, ci, co, kv);
          } else {
            if (w.n_mtile != (ci + 127) / 128) fail("w3 row tiles", es, ci, co, kv);
          }
        }
  std::printf("%d shapes, %d packed weight-gradient plans, %d violations\n", seen, packed, bad);
  return bad ? 1 : 0;
}
