// C ABI and host dispatch of fgms_b200 (see include/fgms_b200.h for the contract of every entry
// point and the reference function each one replaces).  The dispatch plays the role of
// backend/spconv.cu in the reference: it turns (dtype, math, channel counts) into a kernel choice
// and a launch; unlike the reference it validates its arguments, launches on the caller's stream
// and checks the launch status.
#include "../../include/fgms_b200.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"
#include "simt_kernels.cuh"
#include "map_builder.cuh"
#include "umma_gms3.cuh"
#include "umma_wgrad3.cuh"
#include "peer_exchange.cuh"
#include "umma_osfwd.cuh"

namespace {

thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};
// launches that the shape alone would have sent to the tensor-core kernels but that ran on the CUDA-core
// kernels (base pointers not 16-byte aligned): fgms_b200_fallback_count()
std::atomic<long long> g_fallbacks{0};
// SMs the persistent kernels leave free (fgms_b200_set_reserved_sms): room for a kernel of another stream
std::atomic<int> g_reserved_sms{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FGMS_OK;
}

struct DeviceInfo {
  int sms = 0;
  int max_smem_optin = 0;
};

int device_info(DeviceInfo* out) {
  static thread_local int cached_dev = -1;
  static thread_local DeviceInfo cached;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev != cached_dev) {
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    cached.sms = prop.multiProcessorCount;
    cached.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    cached_dev = dev;
  }
  *out = cached;
  const int keep = g_reserved_sms.load(std::memory_order_relaxed);
  if (keep > 0) out->sms = cached.sms - keep > 1 ? cached.sms - keep : 1;
  return FGMS_OK;
}

bool dtype_ok(int dtype) { return dtype == FGMS_DTYPE_F32 || dtype == FGMS_DTYPE_F16; }

int check_math(int dtype, int math) {
  if (!dtype_ok(dtype)) return fail(FGMS_ERR_INVALID_ARG, "unknown dtype %d", dtype);
  if (math != FGMS_MATH_FP32 && math != FGMS_MATH_TF32 && math != FGMS_MATH_F16)
    return fail(FGMS_ERR_INVALID_ARG, "unknown math mode %d", math);
  if (math == FGMS_MATH_TF32 && dtype != FGMS_DTYPE_F32)
    return fail(FGMS_ERR_UNSUPPORTED, "tf32 math needs fp32 storage");
  if (math == FGMS_MATH_F16 && dtype != FGMS_DTYPE_F16)
    return fail(FGMS_ERR_UNSUPPORTED, "f16 math needs fp16 storage");
  return FGMS_OK;
}

int check_dims(int n_in, int n_out, int c_in, int c_out, int k_vol) {
  if (n_in < 0 || n_out < 0) return fail(FGMS_ERR_INVALID_ARG, "negative row count");
  if (c_in < 1 || c_out < 1) return fail(FGMS_ERR_INVALID_ARG, "channel counts must be >= 1");
  if (k_vol < 1 || k_vol > 4096) return fail(FGMS_ERR_INVALID_ARG, "k_vol %d outside [1, 4096]", k_vol);
  if ((long long)k_vol * c_in * c_out >= (1ll << 31)) return fail(FGMS_ERR_INVALID_ARG, "weight tensor too large");
  return FGMS_OK;
}

// Which family a pass of a shape runs on.  One decision for the dispatch and for fgms_b200_kernel_family:
// the tensor-core kernels' own plans (shape rules and shared-memory fit for this k_vol on this device).
bool plan_gms(bool trans, int c_in, int c_out, int k_vol, int dtype, int math, int max_smem) {
  if (math == FGMS_MATH_FP32) return false;
  fgms::G3Config cfg;
  return fgms::g3_plan(c_in, c_out, dtype == FGMS_DTYPE_F16 ? 2 : 4, k_vol, max_smem, trans, &cfg);
}
bool plan_wgrad(int c_in, int c_out, int k_vol, int dtype, int math, int max_smem) {
  if (math == FGMS_MATH_FP32) return false;
  fgms::W3Config cfg;
  return fgms::w3_plan(c_in, c_out, dtype == FGMS_DTYPE_F16 ? 2 : 4, k_vol, max_smem, &cfg);
}

// upper bound on the tiles of `tile` pairs a map of `pairs` entries in k_vol (+1 dense) segments can have
int simt_grid(long long pairs, int dense_rows, int k_vol, int tile, int sms) {
  const long long bound = (pairs + dense_rows) / tile + k_vol + 1;
  const long long full = (long long)sms * 4;
  return (int)(bound < full ? (bound < 1 ? 1 : bound) : full);
}

template <typename T, bool TRANS>
int launch_simt_gms(const fgms::GmsParams& p, cudaStream_t st, int sms) {
  const size_t dyn = (size_t)(2 * p.k_vol + 3) * sizeof(int);
  const int grid = simt_grid(p.pairs, p.dense_rows, p.k_vol, fgms::SIMT_TILE_M, sms);
  if (p.n_dim <= 16) fgms::simt_gms_kernel<T, TRANS, 1><<<grid, fgms::SIMT_THREADS, dyn, st>>>(p);
  else fgms::simt_gms_kernel<T, TRANS, 4><<<grid, fgms::SIMT_THREADS, dyn, st>>>(p);
  return check_launch("simt_gms_kernel");
}

// One gather-GEMM-scatter pass (forward when !trans, dgrad when trans).
int run_gms(bool trans, const void* src, const void* kernel, void* dst, const int32_t* kpos,
            const int32_t* gather_map, const int32_t* scatter_map, int64_t map_len, int n_gather, int n_scatter,
            int c_in, int c_out, int k_vol, int dtype, int math, int dense_rows, int dense_weight,
            cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  fgms::GmsParams p;
  p.src = src; p.weights = kernel; p.dst = dst; p.kpos = kpos;
  p.gather_map = gather_map; p.scatter_map = scatter_map;
  p.pairs = (int)map_len;
  p.n_gather = n_gather; p.n_scatter = n_scatter;
  p.k_dim = trans ? c_out : c_in;
  p.n_dim = trans ? c_in : c_out;
  p.c_in = c_in; p.c_out = c_out; p.k_vol = k_vol;
  p.dense_rows = dense_rows; p.dense_weight = dense_weight;
  if (plan_gms(trans, c_in, c_out, k_vol, dtype, math, di.max_smem_optin)) {
    int rc = fgms::launch_umma_gms3(p, trans, dtype == FGMS_DTYPE_F16, st, di.sms, di.max_smem_optin);
    if (rc == 0) return check_launch("umma_gms3_kernel");
    if (rc < 0) return fail(FGMS_ERR_CUDA, "umma_gms3_kernel setup failed (%d)", rc);
    g_fallbacks.fetch_add(1, std::memory_order_relaxed);  // pointers not 16-byte aligned: CUDA-core path, counted
  }
  if (dtype == FGMS_DTYPE_F16)
    return trans ? launch_simt_gms<__half, true>(p, st, di.sms) : launch_simt_gms<__half, false>(p, st, di.sms);
  return trans ? launch_simt_gms<float, true>(p, st, di.sms) : launch_simt_gms<float, false>(p, st, di.sms);
}

int mid_offset(int k_vol) { return (k_vol % 2 == 1) ? k_vol / 2 : 0; }

// `map_len` is the number of entries in_map and out_map hold.  Kernels clamp every kpos entry to it, so no
// position beyond the maps is read whatever kpos says; maps may be null only when they are empty.
int check_maps(const int32_t* in_map, const int32_t* out_map, int64_t map_len) {
  if (map_len < 0 || map_len > 0x7fffffffll) return fail(FGMS_ERR_INVALID_ARG, "map_len %lld outside [0, 2^31)", (long long)map_len);
  if (map_len > 0 && (!in_map || !out_map)) return fail(FGMS_ERR_INVALID_ARG, "map pointer is null");
  return FGMS_OK;
}

int check_fwd_args(const void* in_feats, const void* kernel, void* out_feats, const int32_t* kpos,
                   const int32_t* in_map, const int32_t* out_map, int64_t map_len, int n_in, int n_out,
                   int c_in, int kernel_c_in, int c_out, int k_vol, int64_t sum_nnz, int dtype, int math,
                   int separate_mid) {
  if (c_in != kernel_c_in)
    return fail(FGMS_ERR_CHANNEL_MISMATCH, "Input feature size and kernel size mismatch");
  if (int rc = check_dims(n_in, n_out, c_in, c_out, k_vol)) return rc;
  if (int rc = check_math(dtype, math)) return rc;
  if (!kernel || !kpos) return fail(FGMS_ERR_INVALID_ARG, "kernel / kpos must not be null");
  if ((n_in > 0 && !in_feats) || (n_out > 0 && !out_feats)) return fail(FGMS_ERR_INVALID_ARG, "feature pointer is null");
  if (sum_nnz < 0) return fail(FGMS_ERR_INVALID_ARG, "sum_nnz is negative");
  if (int rc = check_maps(in_map, out_map, map_len)) return rc;
  if (separate_mid && n_in != n_out)
    return fail(FGMS_ERR_INVALID_ARG, "separate_mid needs n_in == n_out (got %d, %d)", n_in, n_out);
  return FGMS_OK;
}

size_t elem_size(int dtype) { return dtype == FGMS_DTYPE_F16 ? 2 : 4; }

// NVTX range named after the entry point, open for the duration of the host call (the enqueue); a timeline tool
// shows the kernels launched inside it under that name.  Without a tool attached the calls return at once.
struct TraceRange {
  explicit TraceRange(const char* name) { nvtxRangePushA(name); }
  ~TraceRange() { nvtxRangePop(); }
  TraceRange(const TraceRange&) = delete;
  TraceRange& operator=(const TraceRange&) = delete;
};

}  // namespace

extern "C" {

int fgms_b200_fusion_fwd(const void* in_feats, const void* kernel, void* out_feats,
                         const int32_t* kpos, const int32_t* qkpos, const int32_t* in_map,
                         const int32_t* out_map, int64_t map_len, int n_in, int n_out, int c_in,
                         int kernel_c_in, int c_out, int k_vol, int64_t sum_nnz, int dtype, int math,
                         int separate_mid, void* stream) {
  TraceRange trace_range("fgms_b200_fusion_fwd");
  (void)qkpos;
  if (int rc = check_fwd_args(in_feats, kernel, out_feats, kpos, in_map, out_map, map_len, n_in, n_out, c_in,
                              kernel_c_in, c_out, k_vol, sum_nnz, dtype, math, separate_mid))
    return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (separate_mid && n_out > 0) {
    // the reference's centre GEMM runs first with beta = 0: previous contents are discarded
    cudaError_t e = cudaMemsetAsync(out_feats, 0, (size_t)n_out * c_out * elem_size(dtype), st);
    if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  }
  return run_gms(false, in_feats, kernel, out_feats, kpos, in_map, out_map, map_len, n_in, n_out, c_in, c_out,
                 k_vol, dtype, math, separate_mid ? n_in : 0, mid_offset(k_vol), st);
}

int fgms_b200_seq_fwd(const void* in_feats, const void* kernel, void* out_feats,
                      const int32_t* kernel_nnz_host, const int32_t* kpos, const int32_t* in_map,
                      const int32_t* out_map, int64_t map_len, int n_in, int n_out, int c_in,
                      int kernel_c_in, int c_out, int k_vol, int64_t sum_nnz, int dtype, int math,
                      int separate_mid, void* stream) {
  TraceRange trace_range("fgms_b200_seq_fwd");
  if (int rc = check_fwd_args(in_feats, kernel, out_feats, kpos, in_map, out_map, map_len, n_in, n_out, c_in,
                              kernel_c_in, c_out, k_vol, sum_nnz, dtype, math, separate_mid))
    return rc;
  if (!kernel_nnz_host) return fail(FGMS_ERR_INVALID_ARG, "kernel_nnz (host) must not be null");
  long long total = 0;
  for (int k = 0; k < k_vol; ++k) {
    if (kernel_nnz_host[k] < 0) return fail(FGMS_ERR_INVALID_ARG, "kernel_nnz[%d] is negative", k);
    total += kernel_nnz_host[k];
  }
  if (total != sum_nnz)
    return fail(FGMS_ERR_INVALID_ARG, "kernel_nnz sums to %lld but sum_nnz is %lld", total, (long long)sum_nnz);
  if (total > map_len)
    return fail(FGMS_ERR_INVALID_ARG, "kernel_nnz sums to %lld but the maps hold %lld entries", total, (long long)map_len);
  return run_gms(false, in_feats, kernel, out_feats, kpos, in_map, out_map, map_len, n_in, n_out, c_in, c_out,
                 k_vol, dtype, math, separate_mid ? n_in : 0, mid_offset(k_vol),
                 static_cast<cudaStream_t>(stream));
}

int fgms_b200_dgrad(const void* out_grad, const void* kernel, void* in_grad, const int32_t* kpos,
                    const int32_t* in_map, const int32_t* out_map, int64_t map_len, int n_in, int n_out,
                    int c_in, int c_out, int k_vol, int dtype, int math, void* stream) {
  TraceRange trace_range("fgms_b200_dgrad");
  if (int rc = check_dims(n_in, n_out, c_in, c_out, k_vol)) return rc;
  if (int rc = check_math(dtype, math)) return rc;
  if (!kernel || !kpos) return fail(FGMS_ERR_INVALID_ARG, "kernel / kpos must not be null");
  if ((n_out > 0 && !out_grad) || (n_in > 0 && !in_grad)) return fail(FGMS_ERR_INVALID_ARG, "gradient pointer is null");
  if (int rc = check_maps(in_map, out_map, map_len)) return rc;
  return run_gms(true, out_grad, kernel, in_grad, kpos, out_map, in_map, map_len, n_out, n_in, c_in, c_out, k_vol,
                 dtype, math, 0, 0, static_cast<cudaStream_t>(stream));
}

size_t fgms_b200_wgrad_workspace_bytes(int c_in, int c_out, int k_vol, int dtype) {
  if (dtype != FGMS_DTYPE_F16 || c_in < 1 || c_out < 1 || k_vol < 1) return 0;
  return (size_t)k_vol * c_in * c_out * sizeof(float);
}

int fgms_b200_wgrad_finalize(void* kernel_grad_f16, const void* workspace_f32, int64_t count, void* stream) {
  TraceRange trace_range("fgms_b200_wgrad_finalize");
  if (count < 0) return fail(FGMS_ERR_INVALID_ARG, "negative count");
  if (count == 0) return FGMS_OK;
  if (!kernel_grad_f16 || !workspace_f32) return fail(FGMS_ERR_INVALID_ARG, "null pointer");
  int blocks = (int)((count + 255) / 256);
  if (blocks > 1184) blocks = 1184;
  fgms::wgrad_finalize_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__half*>(kernel_grad_f16), static_cast<const float*>(workspace_f32), (long long)count);
  return check_launch("wgrad_finalize_kernel");
}

int fgms_b200_wgrad(const void* in_feats, const void* out_grad, void* kernel_grad,
                    const int32_t* kpos, const int32_t* in_map, const int32_t* out_map, int64_t map_len,
                    int n_in, int n_out, int c_in, int c_out, int k_vol, int dtype, int math,
                    void* workspace, size_t workspace_bytes, int accumulate_into_kernel_grad, void* stream) {
  TraceRange trace_range("fgms_b200_wgrad");
  if (int rc = check_dims(n_in, n_out, c_in, c_out, k_vol)) return rc;
  if (int rc = check_math(dtype, math)) return rc;
  if (!kpos) return fail(FGMS_ERR_INVALID_ARG, "kpos must not be null");
  if (int rc = check_maps(in_map, out_map, map_len)) return rc;
  if ((n_in > 0 && !in_feats) || (n_out > 0 && !out_grad)) return fail(FGMS_ERR_INVALID_ARG, "feature pointer is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  const size_t count = (size_t)k_vol * c_in * c_out;

  float* acc = nullptr;
  // fp16 storage, no workspace: every CTA adds its fp32 partial sums, rounded to fp16, straight into
  // kernel_grad (one launch, no clearing, no second kernel); only the tensor-core kernel does that
  const bool umma = plan_wgrad(c_in, c_out, k_vol, dtype, math, di.max_smem_optin);
  const bool direct_f16 = dtype == FGMS_DTYPE_F16 && workspace == nullptr && accumulate_into_kernel_grad &&
                          kernel_grad != nullptr && umma;
  if (direct_f16) {
    // nothing to prepare
  } else if (dtype == FGMS_DTYPE_F16) {
    const size_t need = fgms_b200_wgrad_workspace_bytes(c_in, c_out, k_vol, dtype);
    if (!workspace || workspace_bytes < need)
      return fail(FGMS_ERR_WORKSPACE, "wgrad needs a %zu-byte workspace for fp16 storage (got %zu)", need,
                  workspace ? workspace_bytes : (size_t)0);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
      return fail(FGMS_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    if (accumulate_into_kernel_grad && !kernel_grad) return fail(FGMS_ERR_INVALID_ARG, "kernel_grad is null");
    cudaError_t e = cudaMemsetAsync(workspace, 0, need, st);
    if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    acc = static_cast<float*>(workspace);
  } else {
    if (!kernel_grad) return fail(FGMS_ERR_INVALID_ARG, "kernel_grad is null");
    acc = static_cast<float*>(kernel_grad);
  }

  fgms::WgradParams p;
  p.feats = in_feats; p.out_grad = out_grad; p.dw = acc; p.kpos = kpos;
  p.in_map = in_map; p.out_map = out_map;
  p.pairs = (int)map_len;
  p.n_in = n_in; p.n_out = n_out; p.c_in = c_in; p.c_out = c_out; p.k_vol = k_vol;
  if (direct_f16) p.dw_f16 = static_cast<__half*>(kernel_grad);

  bool launched = false;
  if (umma) {
    int rc = fgms::launch_umma_wgrad3(p, dtype == FGMS_DTYPE_F16, st, di.sms, di.max_smem_optin);
    if (rc == 0) {
      if (int rc2 = check_launch("umma_wgrad3_kernel")) return rc2;
      launched = true;
    } else if (rc < 0) {
      return fail(FGMS_ERR_CUDA, "umma_wgrad3_kernel setup failed (%d)", rc);
    } else if (direct_f16) {
      return fail(FGMS_ERR_WORKSPACE, "the single-launch fp16 weight gradient needs 16-byte aligned tensors: pass a workspace");
    } else {
      g_fallbacks.fetch_add(1, std::memory_order_relaxed);  // pointers not 16-byte aligned: CUDA-core path, counted
    }
  }
  if (!launched) {
    const size_t dyn = (size_t)(2 * k_vol + 3) * sizeof(int);
    const int grid = simt_grid(map_len, 0, k_vol, fgms::SIMT_WG_TILE, di.sms);
    const bool small = c_in <= 16 && c_out <= 16;
    if (dtype == FGMS_DTYPE_F16) {
      if (small) fgms::simt_wgrad_kernel<__half, 1><<<grid, fgms::SIMT_THREADS, dyn, st>>>(p);
      else fgms::simt_wgrad_kernel<__half, 4><<<grid, fgms::SIMT_THREADS, dyn, st>>>(p);
    } else {
      if (small) fgms::simt_wgrad_kernel<float, 1><<<grid, fgms::SIMT_THREADS, dyn, st>>>(p);
      else fgms::simt_wgrad_kernel<float, 4><<<grid, fgms::SIMT_THREADS, dyn, st>>>(p);
    }
    if (int rc = check_launch("simt_wgrad_kernel")) return rc;
  }
  if (dtype == FGMS_DTYPE_F16 && accumulate_into_kernel_grad && !direct_f16)
    return fgms_b200_wgrad_finalize(kernel_grad, workspace, (int64_t)count, stream);
  return FGMS_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free weight gradient (see the header for who needs it).  The fp32 partial sums live
// in this file-scope device array.  In host code `g_noalloc_scratch` is only a handle for the
// symbol, not a device address: the address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what kernels get.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_noalloc_scratch[FGMS_NOALLOC_MAX_ELEMS];

static int noalloc_scratch(float** out) {
  static std::atomic<float*> cached[64];  // per device ordinal; any thread may call
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(FGMS_ERR_CUDA, "device ordinal %d out of range", dev);
  float* addr = cached[dev].load(std::memory_order_acquire);
  if (!addr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);  // `dev` is current: this is ITS copy of the array
    if (e != cudaSuccess || !p) return fail(FGMS_ERR_CUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    addr = static_cast<float*>(p);
    cached[dev].store(addr, std::memory_order_release);  // two threads racing here store the same address
  }
  *out = addr;
  return FGMS_OK;
}

int fgms_b200_wgrad_f16_noalloc(const void* in_feats, const void* out_grad, void* kernel_grad,
                                const int32_t* kpos, const int32_t* in_map, const int32_t* out_map,
                                int64_t map_len, int n_in, int n_out, int c_in, int c_out, int k_vol,
                                int math, void* stream) {
  TraceRange trace_range("fgms_b200_wgrad_f16_noalloc");
  if (int rc = check_dims(n_in, n_out, c_in, c_out, k_vol)) return rc;
  const long long elems = (long long)k_vol * c_in * c_out;
  if (elems > (long long)FGMS_NOALLOC_MAX_ELEMS)
    return fail(FGMS_ERR_WORKSPACE,
                "k_vol*c_in*c_out = %lld exceeds the %d fp32 values of the built-in scratch array; "
                "call fgms_b200_wgrad with a workspace instead", elems, (int)FGMS_NOALLOC_MAX_ELEMS);
  if (int rc = check_maps(in_map, out_map, map_len)) return rc;
  float* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  // fgms_b200_wgrad clears the first `elems` values itself (cudaMemsetAsync on `stream`)
  return fgms_b200_wgrad(in_feats, out_grad, kernel_grad, kpos, in_map, out_map, map_len, n_in, n_out, c_in,
                         c_out, k_vol, FGMS_DTYPE_F16, math, scratch, (size_t)elems * sizeof(float), 1, stream);
}

int fgms_b200_bwd(const void* out_grad, const void* in_feats, const void* kernel, void* in_grad,
                  void* kernel_grad, const int32_t* kpos, const int32_t* qkpos,
                  const int32_t* in_map, const int32_t* out_map, int64_t map_len, int n_in, int n_out,
                  int c_in, int kernel_c_in, int c_out, int k_vol, int64_t sum_nnz, int dtype, int math,
                  int separate_mid, void* workspace, size_t workspace_bytes, void* stream) {
  TraceRange trace_range("fgms_b200_bwd");
  (void)qkpos; (void)separate_mid;
  if (c_in != kernel_c_in)
    return fail(FGMS_ERR_CHANNEL_MISMATCH, "Input feature size and kernel size mismatch");
  if (sum_nnz < 0) return fail(FGMS_ERR_INVALID_ARG, "sum_nnz is negative");
  if (int rc = fgms_b200_dgrad(out_grad, kernel, in_grad, kpos, in_map, out_map, map_len, n_in, n_out, c_in,
                               c_out, k_vol, dtype, math, stream))
    return rc;
  return fgms_b200_wgrad(in_feats, out_grad, kernel_grad, kpos, in_map, out_map, map_len, n_in, n_out, c_in,
                         c_out, k_vol, dtype, math, workspace, workspace_bytes, 1, stream);
}

int fgms_b200_kernel_family(int pass, int c_in, int c_out, int k_vol, int dtype, int math) {
  if (pass < 0 || pass > 2 || !dtype_ok(dtype) || k_vol < 1) return fail(FGMS_ERR_INVALID_ARG, "bad pass, dtype or k_vol");
  // the current device's opt-in shared memory decides the fit; without a device, that of sm_100 (227 KB)
  DeviceInfo di;
  const int max_smem = device_info(&di) == FGMS_OK ? di.max_smem_optin : 232448;
  if (pass == 2) return plan_wgrad(c_in, c_out, k_vol, dtype, math, max_smem) ? 1 : 0;
  return plan_gms(pass == 1, c_in, c_out, k_vol, dtype, math, max_smem) ? 1 : 0;
}

int64_t fgms_b200_fallback_count(void) { return g_fallbacks.load(std::memory_order_relaxed); }

int fgms_b200_set_reserved_sms(int n) {
  if (n < 0 || n > 64) return fail(FGMS_ERR_INVALID_ARG, "reserved SM count %d outside [0, 64]", n);
  g_reserved_sms.store(n, std::memory_order_relaxed);
  return FGMS_OK;
}

// ---------------------------------------------------------------------------------------------
// Kernel maps (csrc/map_builder.cuh)
// ---------------------------------------------------------------------------------------------
size_t fgms_b200_map_workspace_bytes(int n, int n_cols, int k_vol) {
  if (n < 0 || n_cols < 0 || k_vol < 1) return 0;
  return fgms::maps::layout(n, n_cols, k_vol).total;
}

namespace {
struct MapWs {
  fgms::maps::Layout L;
  uint8_t* base;
  fgms::maps::Table table() const {
    return fgms::maps::Table{reinterpret_cast<unsigned long long*>(base + L.keys), reinterpret_cast<int*>(base + L.vals), L.cap - 1};
  }
  int* dense() const { return reinterpret_cast<int*>(base + L.dense); }
  int* tile_sums() const { return reinterpret_cast<int*>(base + L.tile_sums); }
  int* counter() const { return reinterpret_cast<int*>(base + L.counter); }
};
int map_ws(int n, int n_cols, int k_vol, void* workspace, size_t bytes, MapWs* w) {
  w->L = fgms::maps::layout(n, n_cols, k_vol);
  if (!workspace || bytes < w->L.total)
    return fail(FGMS_ERR_WORKSPACE, "map builder needs a %zu-byte workspace (got %zu)", w->L.total, workspace ? bytes : (size_t)0);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(FGMS_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  w->base = static_cast<uint8_t*>(workspace);
  return FGMS_OK;
}
int blocks_for(long long n, int threads) { return (int)((n + threads - 1) / threads); }
int cuda_fail(const char* what) {
  cudaError_t e = cudaGetLastError();
  return fail(FGMS_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}
}  // namespace

int fgms_b200_build_submanifold_map(const int32_t* coords, int n, int kernel_size, int32_t* kpos, int32_t* in_map,
                                    int32_t* out_map, void* workspace, size_t workspace_bytes, int64_t* pairs_host,
                                    void* stream) {
  TraceRange trace_range("fgms_b200_build_submanifold_map");
  if (n < 0 || kernel_size < 1 || kernel_size > 7 || kernel_size % 2 == 0)
    return fail(FGMS_ERR_INVALID_ARG, "n must be >= 0 and kernel_size odd, 1..7");
  if (!kpos || (n > 0 && (!coords || !in_map || !out_map))) return fail(FGMS_ERR_INVALID_ARG, "null pointer");
  const int k_vol = kernel_size * kernel_size * kernel_size;
  if ((long long)k_vol * n > 0x7fffffffll) return fail(FGMS_ERR_INVALID_ARG, "k_vol * n exceeds the int32 range of the maps");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MapWs w;
  if (int rc = map_ws(n, n, k_vol, workspace, workspace_bytes, &w)) return rc;
  if (n == 0) {
    if (cudaMemsetAsync(kpos, 0, (size_t)(k_vol + 1) * 4, st) != cudaSuccess) return cuda_fail("cudaMemsetAsync");
  } else {
    if (cudaMemsetAsync(w.base + w.L.keys, 0xff, (size_t)w.L.cap * 8, st) != cudaSuccess ||
        cudaMemsetAsync(w.base + w.L.vals, 0x7f, (size_t)w.L.cap * 4, st) != cudaSuccess)
      return cuda_fail("cudaMemsetAsync");
    fgms::maps::insert_kernel<<<blocks_for(n, 256), 256, 0, st>>>(coords, n, 1, w.table(), w.counter());
    const long long cells = (long long)k_vol * n;
    fgms::maps::submanifold_fill_kernel<<<blocks_for(cells, 256), 256, 0, st>>>(coords, n, kernel_size, w.table(), w.dense());
    if (!fgms::maps::finish(w.dense(), k_vol, n, w.tile_sums(), kpos, in_map, out_map, st)) return cuda_fail("map builder launch");
    g_launches += 5;
  }
  if (pairs_host) {
    int32_t total = 0;
    if (cudaMemcpyAsync(&total, kpos + k_vol, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
      return cuda_fail("reading the pair count");
    *pairs_host = total;
  }
  return FGMS_OK;
}

int fgms_b200_build_strided_map(const int32_t* coords, int n, int stride, int32_t* out_coords, int32_t* kpos,
                                int32_t* in_map, int32_t* out_map, void* workspace, size_t workspace_bytes,
                                int* n_out_host, void* stream) {
  TraceRange trace_range("fgms_b200_build_strided_map");
  if (n < 0 || stride < 2 || stride > 4) return fail(FGMS_ERR_INVALID_ARG, "n must be >= 0 and stride 2..4");
  if (!kpos || !n_out_host || (n > 0 && (!coords || !out_coords || !in_map || !out_map)))
    return fail(FGMS_ERR_INVALID_ARG, "null pointer");
  const int k_vol = stride * stride * stride;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MapWs w;
  if (int rc = map_ws(n, n, k_vol, workspace, workspace_bytes, &w)) return rc;
  *n_out_host = 0;
  if (n == 0) {
    if (cudaMemsetAsync(kpos, 0, (size_t)(k_vol + 1) * 4, st) != cudaSuccess) return cuda_fail("cudaMemsetAsync");
    return FGMS_OK;
  }
  auto* ukeys = reinterpret_cast<unsigned long long*>(w.base + w.L.ukeys);
  auto* sorted = reinterpret_cast<unsigned long long*>(w.base + w.L.ukeys_sorted);
  if (cudaMemsetAsync(w.base + w.L.keys, 0xff, (size_t)w.L.cap * 8, st) != cudaSuccess ||
      cudaMemsetAsync(w.counter(), 0, 8, st) != cudaSuccess)
    return cuda_fail("cudaMemsetAsync");
  // unique parents -> counter[0]; their keys, gathered in table order -> counter[1] counts them again
  fgms::maps::insert_kernel<<<blocks_for(n, 256), 256, 0, st>>>(coords, n, stride, w.table(), w.counter());
  fgms::maps::collect_keys_kernel<<<blocks_for(w.L.cap, 256), 256, 0, st>>>(w.table(), ukeys, w.counter() + 1);
  int n_out = 0;
  if (cudaMemcpyAsync(&n_out, w.counter(), 4, cudaMemcpyDeviceToHost, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess)
    return cuda_fail("reading the number of output voxels");
  if (n_out < 1 || n_out > n) return fail(FGMS_ERR_DEVICE, "no output voxel could be formed (coordinates out of range?)");
  size_t cub_bytes = w.L.cub_bytes;
  if (cub::DeviceRadixSort::SortKeys(w.base + w.L.cub, cub_bytes, ukeys, sorted, n_out, 0, 3 * fgms::maps::COORD_BITS, st) != cudaSuccess)
    return cuda_fail("radix sort");
  fgms::maps::rank_kernel<<<blocks_for(n_out, 256), 256, 0, st>>>(sorted, n_out, w.table(), out_coords);
  const long long cells = (long long)k_vol * n_out;
  fgms::maps::fill_kernel<<<blocks_for(cells, 256) < 2048 ? blocks_for(cells, 256) : 2048, 256, 0, st>>>(w.dense(), cells, -1);
  fgms::maps::strided_fill_kernel<<<blocks_for(n, 256), 256, 0, st>>>(coords, n, stride, n_out, w.table(), w.dense());
  if (!fgms::maps::finish(w.dense(), k_vol, n_out, w.tile_sums(), kpos, in_map, out_map, st)) return cuda_fail("map builder launch");
  g_launches += 8;
  *n_out_host = n_out;
  return FGMS_OK;
}

int fgms_b200_transpose_map(const int32_t* kpos, const int32_t* in_map, const int32_t* out_map, int n_in, int k_vol,
                            int64_t pairs, int32_t* kpos_t, int32_t* in_map_t, int32_t* out_map_t, void* workspace,
                            size_t workspace_bytes, void* stream) {
  TraceRange trace_range("fgms_b200_transpose_map");
  if (n_in < 0 || k_vol < 1 || pairs < 0) return fail(FGMS_ERR_INVALID_ARG, "negative size");
  if (!kpos || !kpos_t || (pairs > 0 && (!in_map || !out_map || !in_map_t || !out_map_t)))
    return fail(FGMS_ERR_INVALID_ARG, "null pointer");
  if ((long long)k_vol * n_in > 0x7fffffffll) return fail(FGMS_ERR_INVALID_ARG, "k_vol * n_in exceeds the int32 range of the maps");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MapWs w;
  if (int rc = map_ws(0, n_in, k_vol, workspace, workspace_bytes, &w)) return rc;
  const long long cells = (long long)k_vol * n_in;
  if (cells > 0) fgms::maps::fill_kernel<<<blocks_for(cells, 256) < 2048 ? blocks_for(cells, 256) : 2048, 256, 0, st>>>(w.dense(), cells, -1);
  if (pairs > 0)
    fgms::maps::transpose_fill_kernel<<<blocks_for(pairs, 256), 256, 0, st>>>(kpos, in_map, out_map, k_vol, pairs, n_in, w.dense());
  if (!fgms::maps::finish(w.dense(), k_vol, n_in, w.tile_sums(), kpos_t, in_map_t, out_map_t, st)) return cuda_fail("map builder launch");
  g_launches += 5;
  return FGMS_OK;
}

// ---------------------------------------------------------------------------------------------
// Sum of the ranks' weight-gradient partial sums over peer memory (csrc/peer_exchange.cuh)
// ---------------------------------------------------------------------------------------------
size_t fgms_b200_peer_exchange_flag_bytes(int world) {
  if (world < 1 || world > fgms::PX_MAX_WORLD) return 0;
  return (((size_t)(2 * world + 1) * sizeof(uint32_t)) + 255) & ~(size_t)255;
}

int fgms_b200_peer_exchange(const float* const* sums, float* const* reduced, uint32_t* const* flags, int rank,
                            int world, int64_t count, uint32_t epoch, int64_t wait_limit_cycles, int ctas,
                            void* stream) {
  TraceRange trace_range("fgms_b200_peer_exchange");
  if (world < 1 || world > fgms::PX_MAX_WORLD) return fail(FGMS_ERR_INVALID_ARG, "world %d outside [1, %d]", world, fgms::PX_MAX_WORLD);
  if (rank < 0 || rank >= world) return fail(FGMS_ERR_INVALID_ARG, "rank %d outside [0, %d)", rank, world);
  if (count < 0 || count % 4 != 0) return fail(FGMS_ERR_INVALID_ARG, "count must be a non-negative multiple of 4");
  if (!sums || !reduced || !flags) return fail(FGMS_ERR_INVALID_ARG, "null pointer table");
  if (ctas < 1 || ctas > 1024) return fail(FGMS_ERR_INVALID_ARG, "ctas %d outside [1, 1024]", ctas);
  if (wait_limit_cycles < 0) return fail(FGMS_ERR_INVALID_ARG, "negative wait limit");
  fgms::PeerExchangeParams p = {};
  for (int q = 0; q < world; ++q) {
    if (!flags[q] || (count > 0 && (!sums[q] || !reduced[q]))) return fail(FGMS_ERR_INVALID_ARG, "null buffer of rank %d", q);
    if ((reinterpret_cast<uintptr_t>(sums[q]) | reinterpret_cast<uintptr_t>(reduced[q])) & 15)
      return fail(FGMS_ERR_INVALID_ARG, "buffers of rank %d are not 16-byte aligned", q);
    p.sums[q] = sums[q]; p.reduced[q] = reduced[q]; p.flags[q] = flags[q];
  }
  p.count = count; p.epoch = epoch; p.rank = rank; p.world = world;
  p.wait_limit = wait_limit_cycles > 0 ? wait_limit_cycles : fgms::PX_WAIT_LIMIT_CYCLES;
  // Same shared-memory carve-out as the tensor-core kernels (the largest): an SM keeps ONE carve-out for all the
  // CTAs it holds, so a kernel that prefers another one would wait for the persistent kernel's CTAs to leave.
  static std::atomic<int> carveout_set[64];
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !carveout_set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(fgms::peer_exchange_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared) != cudaSuccess)
      return fail(FGMS_ERR_CUDA, "cudaFuncSetAttribute(carve-out) failed");
    carveout_set[dev].store(1, std::memory_order_release);
  }
  fgms::peer_exchange_kernel<<<ctas, fgms::PX_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch("peer_exchange_kernel");
}

size_t fgms_b200_neighbor_table_bytes(int n_out, int k_vol) {
  if (n_out < 0 || k_vol < 1) return 0;
  return (size_t)k_vol * (((size_t)n_out + fgms::OS_TILE - 1) / fgms::OS_TILE * fgms::OS_TILE) * sizeof(int32_t);
}

int fgms_b200_build_neighbor_table(const int32_t* kpos, const int32_t* in_map, const int32_t* out_map, int64_t map_len,
                                   int n_in, int n_out, int k_vol, int32_t* nbr, size_t nbr_bytes, void* stream) {
  TraceRange trace_range("fgms_b200_build_neighbor_table");
  if (n_in < 0 || n_out < 0 || k_vol < 1 || k_vol > 4096) return fail(FGMS_ERR_INVALID_ARG, "negative row count or k_vol outside [1, 4096]");
  if (!kpos) return fail(FGMS_ERR_INVALID_ARG, "kpos must not be null");
  if (int rc = check_maps(in_map, out_map, map_len)) return rc;
  const size_t need = fgms_b200_neighbor_table_bytes(n_out, k_vol);
  if (need == 0) return FGMS_OK;
  if (!nbr || nbr_bytes < need) return fail(FGMS_ERR_WORKSPACE, "neighbour table needs %zu bytes", need);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(nbr, 0xFF, need, st);  // -1 everywhere: no neighbour
  if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  if (map_len == 0) return FGMS_OK;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  const long long stride = (long long)(need / sizeof(int32_t) / (size_t)k_vol);
  long long blocks = (map_len + 255) / 256;
  if (blocks > 4ll * di.sms) blocks = 4ll * di.sms;
  fgms::os_fill_nbr_kernel<<<(int)blocks, 256, (size_t)(k_vol + 1) * sizeof(int), st>>>(kpos, in_map, out_map, (long long)map_len,
                                                                                         n_in, n_out, k_vol, stride, nbr);
  return check_launch("os_fill_nbr_kernel");
}

int fgms_b200_fwd_output_stationary(const void* in_feats, const void* kernel, void* out_feats, const int32_t* nbr,
                                    int n_in, int n_out, int c_in, int c_out, int k_vol, int dtype, int math,
                                    const void* bias, int relu, int accumulate, void* stream) {
  TraceRange trace_range("fgms_b200_fwd_output_stationary");
  if (int rc = check_dims(n_in, n_out, c_in, c_out, k_vol)) return rc;
  if (int rc = check_math(dtype, math)) return rc;
  if (!kernel) return fail(FGMS_ERR_INVALID_ARG, "kernel must not be null");
  if ((n_in > 0 && !in_feats) || (n_out > 0 && (!out_feats || !nbr))) return fail(FGMS_ERR_INVALID_ARG, "feature or table pointer is null");
  if (accumulate && (bias || relu)) return fail(FGMS_ERR_INVALID_ARG, "bias / ReLU apply to a finished row: not with accumulate");
  if (n_out == 0) return FGMS_OK;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  if (!plan_gms(false, c_in, c_out, k_vol, dtype, math, di.max_smem_optin))
    return fail(FGMS_ERR_UNSUPPORTED, "the output-stationary forward exists for the tensor-core shapes only "
                "(tf32 / fp16 arithmetic, channel counts multiples of 16 up to 256)");
  fgms::OsParams p;
  p.src = in_feats; p.weights = kernel; p.dst = out_feats; p.nbr = nbr; p.bias = bias;
  p.n_tiles = (n_out + fgms::OS_TILE - 1) / fgms::OS_TILE;
  p.nbr_stride = (long long)p.n_tiles * fgms::OS_TILE;
  p.n_in = n_in; p.n_out = n_out; p.c_in = c_in; p.c_out = c_out; p.k_vol = k_vol;
  p.relu = relu ? 1 : 0; p.accumulate = accumulate ? 1 : 0;
  const int rc = fgms::launch_umma_osfwd(p, dtype == FGMS_DTYPE_F16, static_cast<cudaStream_t>(stream), di.sms, di.max_smem_optin);
  if (rc == 0) return check_launch("umma_osfwd_kernel");
  if (rc < 0) return fail(FGMS_ERR_CUDA, "umma_osfwd_kernel setup failed (%d)", rc);
  return fail(FGMS_ERR_INVALID_ARG, "tensors must be 16-byte aligned");
}

int64_t fgms_b200_device_status(int reset) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
  unsigned long long v = 0;
  e = cudaMemcpyFromSymbol(&v, fgms::g_device_problems, sizeof(v));
  if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
  if (reset) {
    unsigned long long z = 0;
    e = cudaMemcpyToSymbol(fgms::g_device_problems, &z, sizeof(z));
    if (e != cudaSuccess) return fail(FGMS_ERR_CUDA, "cudaMemcpyToSymbol: %s", cudaGetErrorString(e));
  }
  return (int64_t)v;
}

int64_t fgms_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* fgms_b200_last_error(void) { return g_err; }

const char* fgms_b200_version(void) { return "fgms_b200 0.2 (sm_100a)"; }

}  // extern "C"
