/*
 * fgms_b200 — C ABI of the B200-native sparse-convolution backend.
 *
 * Drop-in boundary for the operator surface of hkeee21/FGMS (backend/pybind_cuda.cpp:7-11,
 * prototypes backend/spconv.h:10-49).  The reference binds three C++ functions that take
 * at::Tensor handles; this library exposes the same three operations on plain device
 * pointers and sizes, so that any binding layer (ctypes, pybind11, cgo, JNI ...) can call
 * them without linking PyTorch.  All pointers are DEVICE pointers unless a parameter says
 * otherwise; all matrices are dense row-major and contiguous.
 *
 *   in_feats   [n_in , c_in ]             features of the input voxels
 *   kernel     [k_vol, c_in, c_out]       one weight matrix per kernel offset
 *   out_feats  [n_out, c_out]             accumulated into (caller zeroes it)
 *   kpos       int32 [k_vol + 1]          start of each offset's slice of the maps
 *   in_map / out_map  int32 [map_len]     flat, offset-major (input row, output row) pairs
 *   map_len                               entries each of the two maps holds (>= kpos[k_vol])
 *
 * Nothing read from device memory is trusted with an address: every kpos entry is clamped to
 * [0, map_len] before it positions a map read, and a map entry outside [0, n_in) / [0, n_out) makes
 * its pair a no-op.  Both are counted (fgms_b200_device_status); results are then incomplete.
 *
 * Every function returns FGMS_OK (0) or a negative FGMS_ERR_* code and never throws; the
 * text of the last error of the calling thread is available from fgms_b200_last_error().
 * Kernels are enqueued on `stream` (a cudaStream_t passed as void*; NULL = legacy default
 * stream, which is what the reference always uses, backend/spconv.cu:73) and the call
 * returns without synchronising, like the reference.
 *
 * Every entry point that launches work opens an NVTX range named after itself for the duration of the
 * host call, so that a timeline tool shows forward / dgrad / wgrad / exchange by name; without a tool
 * attached the range calls return at once.
 */
#ifndef FGMS_B200_H_
#define FGMS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FGMS_OK 0
#define FGMS_ERR_INVALID_ARG (-1)      /* null pointer, negative size, unknown enum */
#define FGMS_ERR_CHANNEL_MISMATCH (-2) /* "Input feature size and kernel size mismatch" (backend/spconv.cu:39-43) */
#define FGMS_ERR_UNSUPPORTED (-3)      /* dtype/math combination that does not exist */
#define FGMS_ERR_CUDA (-4)             /* a CUDA runtime call or launch failed */
#define FGMS_ERR_WORKSPACE (-5)        /* workspace missing or too small */
#define FGMS_ERR_DEVICE (-6)           /* a kernel reported a problem (bad map index, wait limit hit) */

/* storage type of in_feats / kernel / out_feats (the reference decides on in_feats.scalar_type(),
 * backend/spconv.cu:47-48) */
#define FGMS_DTYPE_F32 0
#define FGMS_DTYPE_F16 1

/* arithmetic of the per-offset contraction.  Accumulation is always fp32.
 *   FP32 : CUDA-core FFMA on the stored values (fp16 storage is widened exactly) — the
 *          reference's arch80 == false fp32 path (backend/spconv.cu:221-228); also the path taken
 *          for channel counts the tensor-core kernels do not cover.
 *   TF32 : tcgen05 kind::tf32 on fp32 storage — the reference's arch80 == true fp32 path
 *          (backend/spconv.cu:213-220, wmma m16n16k8 there).
 *   F16  : tcgen05 kind::f16 on fp16 storage — the reference's fp16 path
 *          (backend/spconv.cu:108-201, wmma m16n16k16 with fp16 accumulators there). */
#define FGMS_MATH_FP32 0
#define FGMS_MATH_TF32 1
#define FGMS_MATH_F16 2

/* Fused forward:  out[out_map[j]] += in[in_map[j]] . kernel[k(j)]  for every pair j.
 * Replaces ConvolutionForwardFused (backend/spconv.cu:23-246; Python name fgms_fusion_fwd_cuda).
 * `qkpos` (the 256-padded prefix sums of cpu-check.py:6-14) and `sum_nnz` (= qkpos[k_vol]) belong
 * to the reference's tiling contract; this library tiles from `kpos` alone and accepts
 * qkpos == NULL.  separate_mid != 0: the centre offset (k_vol/2 for odd k_vol, else 0) is applied
 * densely to all rows (requires n_in == n_out and maps without centre pairs) and, as in the
 * reference (beta = 0, backend/spconv.cu:55-56,76-106), out_feats is OVERWRITTEN, not accumulated. */
int fgms_b200_fusion_fwd(const void* in_feats, const void* kernel, void* out_feats,
                         const int32_t* kpos, const int32_t* qkpos, const int32_t* in_map,
                         const int32_t* out_map, int64_t map_len, int n_in, int n_out, int c_in,
                         int kernel_c_in, int c_out, int k_vol, int64_t sum_nnz, int dtype, int math,
                         int separate_mid, void* stream);

/* Per-offset ("sequential") forward.  Replaces ConvolutionForward (backend/spconv.cu:249-411;
 * Python name fgms_fwd_cuda).  `kernel_nnz_host` is a HOST array of k_vol counts, as in the
 * reference (backend/spconv.cu:308); it is checked against sum_nnz and otherwise unused because
 * the same single-launch kernel runs.  separate_mid adds the dense centre term to out_feats
 * (beta = 1, backend/spconv.cu:282-283,378-410) without overwriting. */
int fgms_b200_seq_fwd(const void* in_feats, const void* kernel, void* out_feats,
                      const int32_t* kernel_nnz_host, const int32_t* kpos, const int32_t* in_map,
                      const int32_t* out_map, int64_t map_len, int n_in, int n_out, int c_in,
                      int kernel_c_in, int c_out, int k_vol, int64_t sum_nnz, int dtype, int math,
                      int separate_mid, void* stream);

/* Input gradient:  in_grad[in_map[j]] += out_grad[out_map[j]] . kernel[k(j)]^T.
 * First launch of ConvolutionBackward (backend/spconv.cu:454-461 fp16, 553-560 tf32). */
int fgms_b200_dgrad(const void* out_grad, const void* kernel, void* in_grad, const int32_t* kpos,
                    const int32_t* in_map, const int32_t* out_map, int64_t map_len, int n_in, int n_out,
                    int c_in, int c_out, int k_vol, int dtype, int math, void* stream);

/* Weight gradient:  kernel_grad[k] += sum over the pairs of offset k of in[in_map[j]]^T (x) out_grad[out_map[j]].
 * Second launch of ConvolutionBackward (backend/spconv.cu:495-548 fp16, 562-569 tf32).
 * Partial sums are accumulated in fp32.  For fp16 storage they live in `workspace`
 * (>= fgms_b200_wgrad_workspace_bytes() bytes, 256-byte aligned device memory, contents
 * ignored on entry; on return it holds the fp32 [k_vol, c_in, c_out] gradient of THIS call, which
 * is what a multi-GPU caller all-reduces) and are then added to kernel_grad; for fp32 storage
 * workspace may be NULL and kernel_grad is accumulated directly.
 * accumulate_into_kernel_grad == 0 leaves kernel_grad untouched (fp16 only): the caller reduces
 * the workspace across ranks and calls fgms_b200_wgrad_finalize itself.
 * fp16 storage with workspace == NULL and accumulate_into_kernel_grad != 0 selects the single-launch
 * form for shapes the tensor-core kernel covers (fgms_b200_kernel_family(2, ...) == 1): every
 * CTA sums its share of an offset's pairs in fp32 and adds that partial sum, rounded to fp16, straight
 * into kernel_grad with fp16 atomics — no clearing, no second kernel, a few fp16 roundings per value
 * (the reference accumulates every product in fp16, backend/spconv.cu:495-548).  Other channel counts
 * return FGMS_ERR_WORKSPACE without a workspace. */
int fgms_b200_wgrad(const void* in_feats, const void* out_grad, void* kernel_grad,
                    const int32_t* kpos, const int32_t* in_map, const int32_t* out_map, int64_t map_len,
                    int n_in, int n_out, int c_in, int c_out, int k_vol, int dtype, int math,
                    void* workspace, size_t workspace_bytes, int accumulate_into_kernel_grad, void* stream);

/* kernel_grad (fp16) += workspace (fp32), element-wise over k_vol * c_in * c_out values. */
int fgms_b200_wgrad_finalize(void* kernel_grad_f16, const void* workspace_f32, int64_t count,
                             void* stream);

size_t fgms_b200_wgrad_workspace_bytes(int c_in, int c_out, int k_vol, int dtype);

/* Weight gradient for fp16 storage that allocates nothing and needs no caller workspace.
 * This entry point has no counterpart in the reference.  It exists for callers that cannot
 * obtain device memory at the time of the call: code running under a memory pool that is already
 * handed out in full, real-time or inference-server threads in which cudaMalloc (a call that may
 * synchronise the whole device) is forbidden, and language bindings that own no allocator at all.
 * It computes exactly what fgms_b200_wgrad computes with accumulate_into_kernel_grad = 1, but the
 * fp32 partial sums live in a fixed array inside the library's device image instead of a
 * caller-provided workspace.
 *   - Limit: k_vol * c_in * c_out <= FGMS_NOALLOC_MAX_ELEMS (2 MiB of fp32; 27 x 128 x 128 fits,
 *     27 x 256 x 128 does not).  Larger shapes are refused with FGMS_ERR_WORKSPACE; use
 *     fgms_b200_wgrad with a workspace for those.  Every GPU that loads the library holds the
 *     2 MiB array until the process exits.
 *   - The first call on each device looks up the array's device address (no allocation).  Make that
 *     first call outside any stream capture.
 *   - All calls on one device share the array; it is cleared at the start of every call.  Two calls
 *     that can overlap on the GPU (different streams, no dependency) race on it: serialise them. */
#define FGMS_NOALLOC_MAX_ELEMS (512 * 1024)
int fgms_b200_wgrad_f16_noalloc(const void* in_feats, const void* out_grad, void* kernel_grad,
                                const int32_t* kpos, const int32_t* in_map, const int32_t* out_map,
                                int64_t map_len, int n_in, int n_out, int c_in, int c_out, int k_vol,
                                int math, void* stream);

/* Both gradients.  Replaces ConvolutionBackward (backend/spconv.cu:414-571; Python name
 * fgms_bwd_cuda).  separate_mid is accepted and ignored, as in the reference. */
int fgms_b200_bwd(const void* out_grad, const void* in_feats, const void* kernel, void* in_grad,
                  void* kernel_grad, const int32_t* kpos, const int32_t* qkpos,
                  const int32_t* in_map, const int32_t* out_map, int64_t map_len, int n_in, int n_out,
                  int c_in, int kernel_c_in, int c_out, int k_vol, int64_t sum_nnz, int dtype, int math,
                  int separate_mid, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Kernel maps on the GPU.  No counterpart in the reference, which loads its maps from files
 * (spconv-test.py:63-73); every caller of the operator needs them, so they are the step right before
 * the path.  Canonical form, identical to what fgms_b200/maps.py builds on the host: offsets
 * enumerated lexicographically over (dx, dy, dz) (the centre is k_vol / 2, backend/spconv.cu:52),
 * pairs offset-major, ascending output row inside an offset.  coords: device int32 [n, 3], every
 * coordinate in [-2^20 + 8, 2^20 - 8), no voxel twice.  kpos: device int32 [k_vol + 1]; in_map /
 * out_map: device int32 with room for the most pairs possible (stated per function).  workspace:
 * 256-byte aligned device memory of fgms_b200_map_workspace_bytes(n, n_cols, k_vol) bytes, where n is
 * the number of voxels that go into the hash table and n_cols the number of output voxels (an upper
 * bound is fine).  Bad coordinates and duplicate voxels are skipped and counted
 * (fgms_b200_device_status).
 * --------------------------------------------------------------------------------------------- */
size_t fgms_b200_map_workspace_bytes(int n, int n_cols, int k_vol);

/* Stride-1 submanifold map, kernel_size odd (3 -> 27 offsets): pair (i, o) belongs to offset d iff
 * coords[i] == coords[o] + d.  in_map / out_map need n * k_vol entries; workspace for (n, n, k_vol).
 * pairs_host, if not NULL, receives kpos[k_vol] (the call then synchronises the stream). */
int fgms_b200_build_submanifold_map(const int32_t* coords, int n, int kernel_size, int32_t* kpos,
                                    int32_t* in_map, int32_t* out_map, void* workspace,
                                    size_t workspace_bytes, int64_t* pairs_host, void* stream);

/* Downsampling map with kernel_size == stride: output voxels are the distinct floor(coords / stride)
 * in lexicographic order, written to out_coords (device int32, room for [n, 3]); the offset of a pair
 * is coords[i] - stride * out_coords[o].  Every input has exactly one pair: in_map / out_map need n
 * entries; workspace for (n, n, stride^3).  The number of output voxels is returned in *n_out_host;
 * the call synchronises the stream once to learn it. */
int fgms_b200_build_strided_map(const int32_t* coords, int n, int stride, int32_t* out_coords,
                                int32_t* kpos, int32_t* in_map, int32_t* out_map, void* workspace,
                                size_t workspace_bytes, int* n_out_host, void* stream);

/* Map of the transposed convolution: the same pairs with input and output swapped, re-ordered to
 * ascending (new) output row inside each offset.  n_in = rows of the ORIGINAL input (the new output);
 * an input row must not occur twice in one offset.  Outputs need `pairs` entries; workspace for
 * (0, n_in, k_vol). */
int fgms_b200_transpose_map(const int32_t* kpos, const int32_t* in_map, const int32_t* out_map,
                            int n_in, int k_vol, int64_t pairs, int32_t* kpos_t, int32_t* in_map_t,
                            int32_t* out_map_t, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Output-stationary forward.  The reference's forward (backend/spconv.cu:23-246, epilogue
 * backend/fwd_kernels.cuh:130-141) and fgms_b200_fusion_fwd add every pair's product to its output row with an
 * atomic: up to k_vol atomics per row in an order that differs from run to run, and nothing can be applied to the
 * finished row inside the kernel.  This entry point computes each output row in one accumulator instead and
 * writes it once, so the result is the same bits on every run and bias + ReLU are applied on the way out:
 *
 *     out[r] = act( sum_k in[nbr[k][r]] * W[k] + bias )      (accumulate = 0)
 *     out[r] += sum_k in[nbr[k][r]] * W[k]                    (accumulate = 1: the reference's contract; no bias, no ReLU)
 *
 * It takes the map as a neighbour table: nbr[k * stride + r] = input row of output row r under offset k, or -1,
 * stride = n_out rounded up to a multiple of 128, fgms_b200_neighbor_table_bytes(n_out, k_vol) bytes in all.
 * fgms_b200_build_neighbor_table fills it from the flat pair list (kpos entries are clamped to map_len, pairs
 * with an entry outside the tensors are skipped and counted); the pair list must hold every output row at most
 * once per offset, as every valid kernel map does.  Tensor-core shapes only (tf32 / f16 math, channel counts
 * multiples of 16 up to 256): FGMS_ERR_UNSUPPORTED otherwise.  `bias`: c_out values of the storage type or
 * NULL.  Cost: one 128-row stage per (128 output rows, offset) however few of those rows have a neighbour
 * there, against one per 128 pairs in the scatter form.  Measured on a B200 (fp16): 0.9 - 1.1 times the scatter
 * form's time (with the zeroing of the output that form needs) on fully occupied grids (26 pairs per voxel), 2.6
 * times on an indoor surface (9.5 pairs per voxel), 8 times on a LiDAR sweep (2.1 pairs per voxel): the form to use where reproducible bits or the fused
 * epilogue are worth that. */
size_t fgms_b200_neighbor_table_bytes(int n_out, int k_vol);
int fgms_b200_build_neighbor_table(const int32_t* kpos, const int32_t* in_map, const int32_t* out_map, int64_t map_len,
                                   int n_in, int n_out, int k_vol, int32_t* nbr, size_t nbr_bytes, void* stream);
int fgms_b200_fwd_output_stationary(const void* in_feats, const void* kernel, void* out_feats, const int32_t* nbr,
                                    int n_in, int n_out, int c_in, int c_out, int k_vol, int dtype, int math,
                                    const void* bias, int relu, int accumulate, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Multi-GPU: sum of the ranks' fp32 weight-gradient partial sums over peer memory.  No counterpart in the
 * reference (it has no multi-GPU path); it stands where a data-parallel caller would otherwise issue an
 * all-reduce of the [k_vol, c_in, c_out] fp32 sums that fgms_b200_wgrad leaves in its workspace.
 * One call per rank and step, one process per GPU.  `sums`, `reduced` and `flags` are HOST arrays of `world`
 * DEVICE pointers, index = rank: entry q is rank q's buffer as mapped into THIS process (peer-mapped memory:
 * CUDA IPC, cuMemMap or a symmetric-memory allocator; entry `rank` is the local buffer).  sums[q] holds rank
 * q's `count` partial sums; on completion reduced[rank] (and every other rank's reduced buffer, written by its
 * owner) holds the totals, added in rank order, the same bits on every rank and run.  flags[q] is
 * fgms_b200_peer_exchange_flag_bytes(world) bytes, zeroed once before the first call.  `epoch` must be
 * larger than that of any earlier call on these buffers and equal on all ranks of one call; with epoch = 0
 * the kernel numbers the calls itself (first call 1, then 2, ...: every rank must then make the same calls with
 * the same `ctas` on these buffers), which lets a launch be replayed from a CUDA graph.
 * The kernel (`ctas` small CTAs; it is meant to run on a side stream beside the input-gradient kernel) waits
 * for the other ranks with a bound of `wait_limit_cycles` SM cycles (0: about one second); a wait that runs
 * out is counted in fgms_b200_device_status, the kernel returns, and the totals of that call are undefined.
 * Only plain loads and stores cross the link. */
size_t fgms_b200_peer_exchange_flag_bytes(int world);
int fgms_b200_peer_exchange(const float* const* sums, float* const* reduced, uint32_t* const* flags, int rank,
                            int world, int64_t count, uint32_t epoch, int64_t wait_limit_cycles, int ctas,
                            void* stream);

/* The tensor-core kernels are persistent: one CTA per SM that holds nearly all of the SM's shared memory and
 * registers, so a kernel of another stream does not start on that SM before they finish.  A caller that wants
 * such a kernel to run BESIDE them (fgms_b200_peer_exchange beside the input gradient, a collective) tells the
 * library to launch on `n` fewer SMs; the setting is process-wide and applies to the launches that follow
 * (set it around the one call it is meant for).  0 restores the full grid.  No counterpart in the reference,
 * whose grids follow the problem size (backend/spconv.cu:111-245). */
int fgms_b200_set_reserved_sms(int n);

/* Which kernel family the dispatch picks for a shape: 0 = CUDA-core (SIMT), 1 = tcgen05.
 * pass: 0 forward, 1 dgrad, 2 wgrad.  The answer comes from the same plan the launch uses (channel
 * counts multiples of 16 and at most 256, and the operands of this k_vol fitting the current device's
 * shared memory), so it is what a call with 16-byte aligned tensors will run.  The reference makes the
 * same choice inside its dispatch and does not expose it (backend/spconv.cu:108-245). */
int fgms_b200_kernel_family(int pass, int c_in, int c_out, int k_vol, int dtype, int math);

/* Number of launches of this process that the plan above put on tcgen05 but that ran on the CUDA-core
 * kernels instead because a tensor's base address was not 16-byte aligned.  Such a call is correct but
 * many times slower; a caller that cares asserts that this stays 0. */
int64_t fgms_b200_fallback_count(void);

/* Device-side problem counter of the current device: number of map entries outside
 * [0, n_in) / [0, n_out) that kernels skipped plus bounded waits that ran out, since the last
 * reset.  Synchronises the device.  Returns the count (>= 0) or a negative FGMS_ERR_*. */
int64_t fgms_b200_device_status(int reset);

/* Number of kernels this library has launched from this process (all threads). */
int64_t fgms_b200_launch_count(void);

const char* fgms_b200_last_error(void);
const char* fgms_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FGMS_B200_H_ */
