// CUDA-core (FFMA) kernels: the true-fp32 arithmetic path and the path for channel counts the
// tensor-core kernels do not cover (not a multiple of 16, or more than 256).  Storage may be fp32 or
// fp16; products are formed and accumulated in fp32.  Every global access is guarded, so any
// c_in / c_out >= 1 and any k_vol is accepted.  Rows are gathered with 16-byte loads whenever the row
// length and the base address allow it (scalar loads otherwise), results leave with 16- or 8-byte
// vector reds.
//
// Role in the reference: the fp32 FFMA forward kernels (_fgms_fusion_fp32*, backend/spconv.cuh:16-665,
// float4 gathers at :509-523) and the scalar fp16 ones (:898-1216).  The reference has no FFMA backward;
// these kernels give it one.
#pragma once

#include "common.cuh"

namespace fgms {

constexpr int SIMT_THREADS = 256;
constexpr int SIMT_TILE_M = 64;  // pairs per tile (forward / dgrad)
constexpr int SIMT_KC = 32;      // contraction chunk held in shared memory

// 16 bytes of T as fp32 values
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
};
template <> struct Vec16<__half> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
};

// rows of `cols` elements starting at `base` can be read 16 bytes at a time from any column that is a
// multiple of Vec16<T>::N
template <typename T>
__device__ __forceinline__ bool rows_vectorisable(const T* base, int cols) {
  return cols % Vec16<T>::N == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
}

// dst[r][0 .. KC) = row(r)[k0 .. k0 + KC) as fp32, zero beyond the row or for row(r) == nullptr.
// `rows` rows, KC = 32 columns, LD = leading dimension of dst.
template <typename T, int LD, typename RowFn>
__device__ __forceinline__ void stage_rows(float* dst, int rows, RowFn row, int k0, int k_dim, bool vec) {
  constexpr int VN = Vec16<T>::N;
  if (vec) {
    constexpr int CPR = SIMT_KC / VN;  // 16-byte chunks per staged row
    for (int e = threadIdx.x; e < rows * CPR; e += SIMT_THREADS) {
      const int r = e / CPR, c = (e % CPR) * VN;
      float v[VN];
#pragma unroll
      for (int i = 0; i < VN; ++i) v[i] = 0.f;
      const T* src = row(r);
      if (src != nullptr && k0 + c < k_dim) Vec16<T>::load(src + k0 + c, v);  // k_dim % VN == 0: the chunk is inside the row
#pragma unroll
      for (int i = 0; i < VN; ++i) dst[r * LD + c + i] = v[i];
    }
  } else {
    for (int e = threadIdx.x; e < rows * SIMT_KC; e += SIMT_THREADS) {
      const int r = e / SIMT_KC, c = e % SIMT_KC;
      const T* src = row(r);
      dst[r * LD + c] = (src != nullptr && k0 + c < k_dim) ? to_float(__ldg(src + k0 + c)) : 0.f;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// forward / dgrad:  dst[scatter_map[j]] += src[gather_map[j]] . B,  B = W_k or W_k^T
// block = 16 x 16 threads, each thread owns 4 rows x TN columns of a 64 x (16*TN) tile.
// When the whole weight matrix is one shared-memory chunk (k_dim <= 32, n_dim <= 16 TN) it stays
// there across consecutive tiles of one offset.
// ---------------------------------------------------------------------------------------------
template <typename T, bool TRANS_W, int TN>
__global__ void __launch_bounds__(SIMT_THREADS) simt_gms_kernel(GmsParams p) {
  constexpr int BN = 16 * TN;
  extern __shared__ int smem_dyn[];
  int* tile_start = smem_dyn;               // [k_vol + 2]
  int* kpos_s = tile_start + p.k_vol + 2;   // [k_vol + 1]
  __shared__ float As[SIMT_TILE_M * (SIMT_KC + 1)];
  __shared__ float Bs[SIMT_KC][BN + 1];
  __shared__ int rows_g[SIMT_TILE_M];
  __shared__ int rows_s[SIMT_TILE_M];

  const T* __restrict__ src = static_cast<const T*>(p.src);
  const T* __restrict__ w = static_cast<const T*>(p.weights);
  T* dst = static_cast<T*>(p.dst);

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int n_seg = p.k_vol + 1;

  build_tile_table(SIMT_TILE_M, p.kpos, p.pairs, p.k_vol, p.dense_rows, kpos_s, tile_start);
  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);

  const bool vec_out = (sizeof(T) == 4) ? (p.n_dim % 4 == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0)
                                        : (p.n_dim % 4 == 0 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0);
  const bool vec_in = rows_vectorisable(src, p.k_dim);
  const bool w_resident = p.k_dim <= SIMT_KC && p.n_dim <= BN;
  int resident_w = -1;

  for (int t = t0; t < t1; ++t) {
    const int seg = find_segment(tile_start, n_seg, t);
    const int lt = t - tile_start[seg];
    const bool dense = seg == p.k_vol;
    const int seg_base = dense ? 0 : kpos_s[seg];
    const int seg_cnt = dense ? p.dense_rows : (kpos_s[seg + 1] - seg_base);
    const int cnt = min(SIMT_TILE_M, seg_cnt - lt * SIMT_TILE_M);
    const int widx = dense ? p.dense_weight : seg;
    const T* __restrict__ wk = w + (size_t)widx * p.c_in * p.c_out;

    __syncthreads();  // previous tile finished with rows_*, As and Bs
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
    auto gathered_row = [&](int r) -> const T* {
      const int g = rows_g[r];
      return g >= 0 ? src + (size_t)g * p.k_dim : nullptr;
    };

    for (int n0 = 0; n0 < p.n_dim; n0 += BN) {
      float acc[4][TN];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < TN; ++c) acc[r][c] = 0.f;

      for (int k0 = 0; k0 < p.k_dim; k0 += SIMT_KC) {
        stage_rows<T, SIMT_KC + 1>(As, SIMT_TILE_M, gathered_row, k0, p.k_dim, vec_in);
        // weight chunk -> Bs[kk][n]
        if (!w_resident || resident_w != widx) {
          if (!TRANS_W) {
            // B[kk][n] = W[k0+kk][n0+n], contiguous along n
            for (int e = tid; e < SIMT_KC * BN; e += SIMT_THREADS) {
              const int kk = e / BN, n = e % BN;
              float v = 0.f;
              if (k0 + kk < p.k_dim && n0 + n < p.n_dim) v = to_float(__ldg(wk + (size_t)(k0 + kk) * p.c_out + n0 + n));
              Bs[kk][n] = v;
            }
          } else {
            // B[kk][n] = W[n0+n][k0+kk], contiguous along kk
            for (int e = tid; e < SIMT_KC * BN; e += SIMT_THREADS) {
              const int n = e / SIMT_KC, kk = e % SIMT_KC;
              float v = 0.f;
              if (k0 + kk < p.k_dim && n0 + n < p.n_dim) v = to_float(__ldg(wk + (size_t)(n0 + n) * p.c_out + k0 + kk));
              Bs[kk][n] = v;
            }
          }
          resident_w = widx;
        }
        __syncthreads();
        const int k_len = min(SIMT_KC, p.k_dim - k0);
        if (k_len == SIMT_KC) {
#pragma unroll
          for (int kk = 0; kk < SIMT_KC; ++kk) {
            float a[4], b[TN];
#pragma unroll
            for (int r = 0; r < 4; ++r) a[r] = As[(ty * 4 + r) * (SIMT_KC + 1) + kk];
#pragma unroll
            for (int c = 0; c < TN; ++c) b[c] = Bs[kk][tx * TN + c];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
              for (int c = 0; c < TN; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
          }
        } else {
          for (int kk = 0; kk < k_len; ++kk) {
            float a[4], b[TN];
#pragma unroll
            for (int r = 0; r < 4; ++r) a[r] = As[(ty * 4 + r) * (SIMT_KC + 1) + kk];
#pragma unroll
            for (int c = 0; c < TN; ++c) b[c] = Bs[kk][tx * TN + c];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
              for (int c = 0; c < TN; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
          }
        }
        if (k0 + SIMT_KC < p.k_dim || n0 + BN < p.n_dim) __syncthreads();  // As / Bs are rewritten in this tile
      }

      const int n = n0 + tx * TN;
      const int valid = min(TN, p.n_dim - n);
      if (valid > 0) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int s = rows_s[ty * 4 + r];
          if (s >= 0) scatter_add<TN>(dst + (size_t)s * p.n_dim + n, acc[r], valid, vec_out);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// wgrad:  dw[k] += sum_j feats[in_map[j]]^T (x) out_grad[out_map[j]]   (fp32 accumulation)
// A CTA owns a contiguous range of 256-pair tiles.  For each run of its tiles inside one offset and
// each (16 TT) x (16 TT) block of dw[k] it walks the run's pairs in chunks of 32, gathers the block's
// columns of both operands once per chunk and keeps the block's sums in registers until the run ends:
// one red per value, run and CTA.  Channel counts up to 16 TT on both sides gather every row exactly once.
// ---------------------------------------------------------------------------------------------
constexpr int SIMT_WG_TILE = 64;   // pairs per scheduling tile (small: a small map still spreads over many CTAs)
constexpr int SIMT_WG_JC = 32;     // pairs per shared-memory chunk

template <typename T, int TT>
__global__ void __launch_bounds__(SIMT_THREADS) simt_wgrad_kernel(WgradParams p) {
  constexpr int BM = 16 * TT;
  constexpr int LD = BM + 1;
  extern __shared__ int smem_dyn[];
  int* tile_start = smem_dyn;
  int* kpos_s = tile_start + p.k_vol + 2;
  __shared__ float As[SIMT_WG_JC * LD];
  __shared__ float Gs[SIMT_WG_JC * LD];
  __shared__ int rows_i[SIMT_WG_JC];
  __shared__ int rows_o[SIMT_WG_JC];

  const T* __restrict__ feats = static_cast<const T*>(p.feats);
  const T* __restrict__ og = static_cast<const T*>(p.out_grad);

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int n_seg = p.k_vol + 1;
  build_tile_table(SIMT_WG_TILE, p.kpos, p.pairs, p.k_vol, 0, kpos_s, tile_start);
  int t0, t1;
  cta_tile_range(tile_start[n_seg], &t0, &t1);
  const bool vec_out = (p.c_out % 4 == 0) && (reinterpret_cast<uintptr_t>(p.dw) & 15) == 0;
  constexpr int VN = Vec16<T>::N;
  const bool vec_a = rows_vectorisable(feats, p.c_in) && BM % VN == 0;
  const bool vec_g = rows_vectorisable(og, p.c_out) && BM % VN == 0;

  // transposed staging: dst[j][c] = row(j)[c0 + c], BM columns, zero beyond the row
  auto stage = [&](float* dst, const T* base, int cols, const int* rows, int c0, bool vec) {
    if (vec) {
      constexpr int CPR = BM / VN;
      for (int e = tid; e < SIMT_WG_JC * CPR; e += SIMT_THREADS) {
        const int j = e / CPR, c = (e % CPR) * VN;
        float v[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) v[i] = 0.f;
        const int r = rows[j];
        if (r >= 0 && c0 + c < cols) Vec16<T>::load(base + (size_t)r * cols + c0 + c, v);
#pragma unroll
        for (int i = 0; i < VN; ++i) dst[j * LD + c + i] = v[i];
      }
    } else {
      for (int e = tid; e < SIMT_WG_JC * BM; e += SIMT_THREADS) {
        const int j = e / BM, c = e % BM;
        const int r = rows[j];
        dst[j * LD + c] = (r >= 0 && c0 + c < cols) ? to_float(__ldg(base + (size_t)r * cols + c0 + c)) : 0.f;
      }
    }
  };

  int t = t0;
  while (t < t1) {
    const int seg = find_segment(tile_start, n_seg, t);
    const int t_end = min(t1, tile_start[seg + 1]);  // this CTA's tiles of the offset end here
    const int seg_base = kpos_s[seg];
    const int seg_cnt = kpos_s[seg + 1] - seg_base;
    const int j_begin = (t - tile_start[seg]) * SIMT_WG_TILE;
    const int j_end = min(seg_cnt, (t_end - tile_start[seg]) * SIMT_WG_TILE);
    float* dwk = p.dw + (size_t)seg * p.c_in * p.c_out;

    for (int m0 = 0; m0 < p.c_in; m0 += BM) {
      for (int n0 = 0; n0 < p.c_out; n0 += BM) {
        float acc[TT][TT];
#pragma unroll
        for (int r = 0; r < TT; ++r)
#pragma unroll
          for (int c = 0; c < TT; ++c) acc[r][c] = 0.f;

        for (int j0 = j_begin; j0 < j_end; j0 += SIMT_WG_JC) {
          __syncthreads();  // the previous chunk has been consumed
          if (tid < SIMT_WG_JC) {
            int i = -1, o = -1;
            if (j0 + tid < j_end) {
              const int j = seg_base + j0 + tid;
              i = __ldg(p.in_map + j);
              o = __ldg(p.out_map + j);
              if (i < 0 || i >= p.n_in || o < 0 || o >= p.n_out) {
                if (m0 == 0 && n0 == 0) report_problem();  // counted once per skipped pair
                i = o = -1;
              }
            }
            rows_i[tid] = i;
            rows_o[tid] = o;
          }
          __syncthreads();
          stage(As, feats, p.c_in, rows_i, m0, vec_a);
          stage(Gs, og, p.c_out, rows_o, n0, vec_g);
          __syncthreads();
#pragma unroll 8
          for (int jj = 0; jj < SIMT_WG_JC; ++jj) {
            float a[TT], g[TT];
#pragma unroll
            for (int r = 0; r < TT; ++r) a[r] = As[jj * LD + ty * TT + r];
#pragma unroll
            for (int c = 0; c < TT; ++c) g[c] = Gs[jj * LD + tx * TT + c];
#pragma unroll
            for (int r = 0; r < TT; ++r)
#pragma unroll
              for (int c = 0; c < TT; ++c) acc[r][c] = fmaf(a[r], g[c], acc[r][c]);
          }
        }

        const int n = n0 + tx * TT;
        const int valid = min(TT, p.c_out - n);
        if (valid > 0) {
#pragma unroll
          for (int r = 0; r < TT; ++r) {
            const int m = m0 + ty * TT + r;
            if (m < p.c_in) scatter_add<TT>(dwk + (size_t)m * p.c_out + n, acc[r], valid, vec_out);
          }
        }
      }
    }
    t = t_end;
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
