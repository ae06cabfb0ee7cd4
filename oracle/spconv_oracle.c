/*
 * Plain-C restatement of the FGMS reference CPU definition.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA path and the timed CPU baseline of the benchmark; the
 * product library never links or calls it.
 *
 * Follows, loop for loop:
 *   forward   cpu_compute   cpu-check.py:16-44       (pair loop, then the optional centre
 *                                                     term when `precompute`, :39-43)
 *   backward  cpu_compute   cpu-check-back.py:16-44  (in_grad and weight_grad together)
 *   centre    mid_k = k_vol/2 for odd k_vol else 0   cpu-check.py:27, backend/spconv.cu:52
 *
 * The *_f32 functions accumulate one fp32 product at a time in the reference's loop order,
 * which is what the reference's Python loop over fp32 torch scalars does; built with
 * -ffp-contract=off they reproduce it bit for bit.  The *_f64 functions take fp32 inputs
 * and accumulate in double: the ground truth the CUDA kernels are compared with.
 *
 * Parity pin: tests/golden/*.npz (outputs of the reference's own unmodified cpu_compute).
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

static int mid_offset(int k_vol) { return (k_vol % 2 == 1) ? k_vol / 2 : 0; }

#define DEFINE_FWD(NAME, ACC)                                                                  \
  void NAME(const float* feats, const float* w, ACC* out, int n_out, int c_in, int c_out,      \
            int k_vol, const int32_t* knnz, const int32_t* imap, const int32_t* omap,          \
            int precompute) {                                                                  \
    memset(out, 0, sizeof(ACC) * (size_t)n_out * (size_t)c_out);                               \
    size_t j = 0;                                                                              \
    for (int k = 0; k < k_vol; ++k) {                                                          \
      const float* wk = w + (size_t)k * c_in * c_out;                                          \
      for (int n = 0; n < knnz[k]; ++n, ++j) {                                                 \
        const float* f = feats + (size_t)imap[j] * c_in;                                       \
        ACC* o = out + (size_t)omap[j] * c_out;                                                \
        for (int co = 0; co < c_out; ++co)                                                     \
          for (int ci = 0; ci < c_in; ++ci) o[co] += (ACC)f[ci] * (ACC)wk[(size_t)ci * c_out + co]; \
      }                                                                                        \
    }                                                                                          \
    if (precompute) {                                                                          \
      const float* wm = w + (size_t)mid_offset(k_vol) * c_in * c_out;                          \
      for (int i = 0; i < n_out; ++i)                                                          \
        for (int co = 0; co < c_out; ++co)                                                     \
          for (int ci = 0; ci < c_in; ++ci)                                                    \
            out[(size_t)i * c_out + co] +=                                                     \
                (ACC)feats[(size_t)i * c_in + ci] * (ACC)wm[(size_t)ci * c_out + co];          \
    }                                                                                          \
  }

#define DEFINE_BWD(NAME, ACC)                                                                  \
  void NAME(const float* out_grad, const float* w, const float* feats, ACC* in_grad,           \
            ACC* w_grad, int n_in, int c_in, int c_out, int k_vol, const int32_t* knnz,        \
            const int32_t* imap, const int32_t* omap) {                                        \
    memset(in_grad, 0, sizeof(ACC) * (size_t)n_in * (size_t)c_in);                             \
    memset(w_grad, 0, sizeof(ACC) * (size_t)k_vol * c_in * c_out);                             \
    size_t j = 0;                                                                              \
    for (int k = 0; k < k_vol; ++k) {                                                          \
      const float* wk = w + (size_t)k * c_in * c_out;                                          \
      ACC* gk = w_grad + (size_t)k * c_in * c_out;                                             \
      for (int n = 0; n < knnz[k]; ++n, ++j) {                                                 \
        const float* f = feats + (size_t)imap[j] * c_in;                                       \
        const float* g = out_grad + (size_t)omap[j] * c_out;                                   \
        ACC* ig = in_grad + (size_t)imap[j] * c_in;                                            \
        for (int ci = 0; ci < c_in; ++ci)                                                      \
          for (int co = 0; co < c_out; ++co) {                                                 \
            ig[ci] += (ACC)g[co] * (ACC)wk[(size_t)ci * c_out + co];                           \
            gk[(size_t)ci * c_out + co] += (ACC)f[ci] * (ACC)g[co];                            \
          }                                                                                    \
      }                                                                                        \
    }                                                                                          \
  }

DEFINE_FWD(fgms_oracle_fwd_f32, float)
DEFINE_FWD(fgms_oracle_fwd_f64, double)
DEFINE_BWD(fgms_oracle_bwd_f32, float)
DEFINE_BWD(fgms_oracle_bwd_f64, double)
