// CUDA-core (FFMA) kernels: the true-fp32 arithmetic path and the path for channel counts the
// tensor-core kernels do not cover (odd, tiny or not a multiple of 128 bytes per row).  Storage may
// be fp32 or fp16; products are formed and accumulated in fp32.  Every global access is guarded,
// so any c_in / c_out >= 1 and any k_vol is accepted.
//
// Role in the reference: the fp32 FFMA forward kernels (_fgms_fusion_fp32*, backend/spconv.cuh:16-665)
// and the scalar fp16 ones (:898-1216).  The reference has no FFMA backward; these kernels give it one.
#pragma once

#include "common.cuh"

namespace fgms {

constexpr int SIMT_THREADS = 256;
constexpr int SIMT_TILE_M = 64;  // pairs per tile (forward / dgrad)
constexpr int SIMT_KC = 32;      // contraction chunk held in shared memory

// ---------------------------------------------------------------------------------------------
// forward / dgrad:  dst[scatter_map[j]] += src[gather_map[j]] . B,  B = W_k or W_k^T
// block = 16 x 16 threads, each thread owns 4 rows x TN columns of a 64 x (16*TN) tile
// ---------------------------------------------------------------------------------------------
template <typename T, bool TRANS_W, int TN>
__global__ void __launch_bounds__(SIMT_THREADS) simt_gms_kernel(GmsParams p) {
  constexpr int BN = 16 * TN;
  extern __shared__ int smem_dyn[];
  int* tile_start = smem_dyn;  // [k_vol + 2]
  __shared__ float As[SIMT_TILE_M][SIMT_KC + 1];
  __shared__ float Bs[SIMT_KC][BN + 1];
  __shared__ int rows_g[SIMT_TILE_M];
  __shared__ int rows_s[SIMT_TILE_M];

  const T* __restrict__ src = static_cast<const T*>(p.src);
  const T* __restrict__ w = static_cast<const T*>(p.weights);
  T* dst = static_cast<T*>(p.dst);

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int n_seg = p.k_vol + 1;

  build_tile_table(SIMT_TILE_M, p.kpos, p.k_vol, p.dense_rows, tile_start);
  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);

  const bool vec = (sizeof(T) == 4) ? (p.n_dim % 4 == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0)
                                    : (p.n_dim % 2 == 0 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0);

  for (int t = t0; t < t1; ++t) {
    const int seg = find_segment(tile_start, n_seg, t);
    const int lt = t - tile_start[seg];
    const bool dense = seg == p.k_vol;
    const int seg_base = dense ? 0 : __ldg(p.kpos + seg);
    const int seg_cnt = dense ? p.dense_rows : (__ldg(p.kpos + seg + 1) - seg_base);
    const int cnt = min(SIMT_TILE_M, seg_cnt - lt * SIMT_TILE_M);
    const int widx = dense ? p.dense_weight : seg;
    const T* __restrict__ wk = w + (size_t)widx * p.c_in * p.c_out;

    __syncthreads();  // previous tile finished with rows_*
    if (tid < SIMT_TILE_M) {
      int g = -1, s = -1;
      if (tid < cnt) {
        const int j = lt * SIMT_TILE_M + tid;
        g = dense ? j : __ldg(p.gather_map + seg_base + j);
        s = dense ? j : __ldg(p.scatter_map + seg_base + j);
        if (g < 0 || g >= p.n_gather || s < 0 || s >= p.n_scatter) {
          report_problem();
          g = s = -1;
        }
      }
      rows_g[tid] = g;
      rows_s[tid] = s;
    }
    __syncthreads();

    for (int n0 = 0; n0 < p.n_dim; n0 += BN) {
      float acc[4][TN];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < TN; ++c) acc[r][c] = 0.f;

      for (int k0 = 0; k0 < p.k_dim; k0 += SIMT_KC) {
        // gathered rows -> As (coalesced along the row)
#pragma unroll
        for (int i = 0; i < SIMT_TILE_M * SIMT_KC / SIMT_THREADS; ++i) {
          const int r = (tid >> 5) + 8 * i, kk = tid & 31;
          const int g = rows_g[r];
          float v = 0.f;
          if (g >= 0 && k0 + kk < p.k_dim) v = to_float(src[(size_t)g * p.k_dim + k0 + kk]);
          As[r][kk] = v;
        }
        // weight chunk -> Bs[kk][n]
        if (!TRANS_W) {
          // B[kk][n] = W[k0+kk][n0+n], contiguous along n
          for (int e = tid; e < SIMT_KC * BN; e += SIMT_THREADS) {
            const int kk = e / BN, n = e % BN;
            float v = 0.f;
            if (k0 + kk < p.k_dim && n0 + n < p.n_dim) v = to_float(wk[(size_t)(k0 + kk) * p.c_out + n0 + n]);
            Bs[kk][n] = v;
          }
        } else {
          // B[kk][n] = W[n0+n][k0+kk], contiguous along kk
          for (int e = tid; e < SIMT_KC * BN; e += SIMT_THREADS) {
            const int n = e / SIMT_KC, kk = e % SIMT_KC;
            float v = 0.f;
            if (k0 + kk < p.k_dim && n0 + n < p.n_dim) v = to_float(wk[(size_t)(n0 + n) * p.c_out + k0 + kk]);
            Bs[kk][n] = v;
          }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SIMT_KC; ++kk) {
          float a[4], b[TN];
#pragma unroll
          for (int r = 0; r < 4; ++r) a[r] = As[ty * 4 + r][kk];
#pragma unroll
          for (int c = 0; c < TN; ++c) b[c] = Bs[kk][tx * TN + c];
#pragma unroll
          for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < TN; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
        }
        __syncthreads();
      }

      const int n = n0 + tx * TN;
      const int valid = min(TN, p.n_dim - n);
      if (valid > 0) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int s = rows_s[ty * 4 + r];
          if (s >= 0) scatter_add<TN>(dst + (size_t)s * p.n_dim + n, acc[r], valid, vec);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// wgrad:  dw[k] += sum_j feats[in_map[j]]^T (x) out_grad[out_map[j]]   (fp32 accumulation)
// block tile (16*TT) x (16*TT) of dw[k]; the CTA walks its pair tiles and, for each, all blocks.
// ---------------------------------------------------------------------------------------------
constexpr int SIMT_WG_TILE = 256;  // pairs per tile
constexpr int SIMT_WG_JC = 16;     // pairs per shared-memory chunk

template <typename T, int TT>
__global__ void __launch_bounds__(SIMT_THREADS) simt_wgrad_kernel(WgradParams p) {
  constexpr int BM = 16 * TT;
  extern __shared__ int smem_dyn[];
  int* tile_start = smem_dyn;
  __shared__ float As[SIMT_WG_JC][BM + 1];
  __shared__ float Gs[SIMT_WG_JC][BM + 1];
  __shared__ int rows_i[SIMT_WG_TILE];
  __shared__ int rows_o[SIMT_WG_TILE];

  const T* __restrict__ feats = static_cast<const T*>(p.feats);
  const T* __restrict__ og = static_cast<const T*>(p.out_grad);

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int n_seg = p.k_vol + 1;
  build_tile_table(SIMT_WG_TILE, p.kpos, p.k_vol, 0, tile_start);
  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);
  const bool vec = (p.c_out % 4 == 0) && (reinterpret_cast<uintptr_t>(p.dw) & 15) == 0;

  for (int t = t0; t < t1; ++t) {
    const int seg = find_segment(tile_start, n_seg, t);
    const int lt = t - tile_start[seg];
    const int seg_base = __ldg(p.kpos + seg);
    const int seg_cnt = __ldg(p.kpos + seg + 1) - seg_base;
    const int cnt = min(SIMT_WG_TILE, seg_cnt - lt * SIMT_WG_TILE);
    float* dwk = p.dw + (size_t)seg * p.c_in * p.c_out;

    __syncthreads();
    for (int r = tid; r < SIMT_WG_TILE; r += SIMT_THREADS) {
      int i = -1, o = -1;
      if (r < cnt) {
        const int j = seg_base + lt * SIMT_WG_TILE + r;
        i = __ldg(p.in_map + j);
        o = __ldg(p.out_map + j);
        if (i < 0 || i >= p.n_in || o < 0 || o >= p.n_out) {
          report_problem();
          i = o = -1;
        }
      }
      rows_i[r] = i;
      rows_o[r] = o;
    }
    __syncthreads();

    for (int m0 = 0; m0 < p.c_in; m0 += BM) {
      for (int n0 = 0; n0 < p.c_out; n0 += BM) {
        float acc[TT][TT];
#pragma unroll
        for (int r = 0; r < TT; ++r)
#pragma unroll
          for (int c = 0; c < TT; ++c) acc[r][c] = 0.f;

        for (int j0 = 0; j0 < cnt; j0 += SIMT_WG_JC) {
          for (int e = tid; e < SIMT_WG_JC * BM; e += SIMT_THREADS) {
            const int jj = e / BM, c = e % BM;
            const int i = rows_i[j0 + jj], o = rows_o[j0 + jj];  // j0 + jj < SIMT_WG_TILE always
            float a = 0.f, g = 0.f;
            if (i >= 0) {
              if (m0 + c < p.c_in) a = to_float(feats[(size_t)i * p.c_in + m0 + c]);
              if (n0 + c < p.c_out) g = to_float(og[(size_t)o * p.c_out + n0 + c]);
            }
            As[jj][c] = a;
            Gs[jj][c] = g;
          }
          __syncthreads();
#pragma unroll
          for (int jj = 0; jj < SIMT_WG_JC; ++jj) {
            float a[TT], g[TT];
#pragma unroll
            for (int r = 0; r < TT; ++r) a[r] = As[jj][ty * TT + r];
#pragma unroll
            for (int c = 0; c < TT; ++c) g[c] = Gs[jj][tx * TT + c];
#pragma unroll
            for (int r = 0; r < TT; ++r)
#pragma unroll
              for (int c = 0; c < TT; ++c) acc[r][c] = fmaf(a[r], g[c], acc[r][c]);
          }
          __syncthreads();
        }

        const int n = n0 + tx * TT;
        const int valid = min(TT, p.c_out - n);
        if (valid > 0) {
#pragma unroll
          for (int r = 0; r < TT; ++r) {
            const int m = m0 + ty * TT + r;
            if (m < p.c_in) scatter_add<TT>(dwk + (size_t)m * p.c_out + n, acc[r], valid, vec);
          }
        }
      }
    }
  }
}

// kernel_grad(fp16) += workspace(fp32)
__global__ void wgrad_finalize_kernel(__half* __restrict__ kg, const float* __restrict__ ws, long long count) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    kg[i] = __float2half_rn(__half2float(kg[i]) + ws[i]);
  }
}

}  // namespace fgms
