"""PyTorch binding with the operator surface of ``FGMS.backend``.

The reference exports three functions from ``backend/pybind_cuda.cpp:8-10`` (prototypes in
``backend/spconv.h:10-49``).  The functions below keep their names, positional signatures,
in-place accumulate semantics and error behaviour, and forward to the C ABI of
``libfgms_b200.so`` with raw device pointers — this file is the only torch-aware layer.

Differences from the reference, all deliberate:

* kernels run on PyTorch's *current* stream, not on the legacy default stream
  (``backend/spconv.cu:73``);
* arguments are validated (device, dtype, contiguity, shapes) and raise ``ValueError`` instead
  of reading out of bounds;
* fp16 products are accumulated in fp32 inside a tile (the reference accumulates in fp16,
  ``backend/fwd_kernels.cuh:66``); what crosses CTAs is added with fp16 atomics like the reference's, except
  in the workspace form of the weight gradient (``WGRAD_FP32_SUMS``), which stays fp32 to the end;
* ``arch80`` selects the arithmetic for fp32 storage in the backward as well as the forward
  (``True`` → tf32 tensor cores, ``False`` → exact fp32 FFMA); the reference's backward ignores
  the flag and always uses tf32 (``backend/spconv.cu:551-570``).
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["fgms_fusion_fwd_cuda", "fgms_fwd_cuda", "fgms_bwd_cuda", "fgms_dgrad_cuda", "fgms_wgrad_cuda",
           "wgrad_workspace", "wgrad_finalize", "fgms_wgrad_noalloc_cuda", "kernel_family", "fallback_count",
           "device_status", "launch_count", "build_neighbor_table", "fgms_fwd_os_cuda"]

_L = _lib.lib


def _dtype_math(t: torch.Tensor, arch80: bool):
    if t.dtype == torch.float16:
        return _lib.DTYPE_F16, _lib.MATH_F16
    if t.dtype == torch.float32:
        return _lib.DTYPE_F32, (_lib.MATH_TF32 if arch80 else _lib.MATH_FP32)
    raise ValueError(f"unsupported feature dtype {t.dtype}: the operator takes float16 or float32")


def _check_feat(name, t, dtype=None, dim=2):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dim() != dim:
        raise ValueError(f"{name} must have {dim} dimensions, got {t.dim()}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")


def _check_index(name, t, device, min_len=None, cuda=True):
    if not isinstance(t, torch.Tensor) or t.dtype != torch.int32:
        raise ValueError(f"{name} must be an int32 tensor")
    if cuda and (not t.is_cuda or t.device != device):
        raise ValueError(f"{name} must live on {device}")
    if not cuda and t.is_cuda:
        raise ValueError(f"{name} must be a CPU tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if min_len is not None and t.numel() < min_len:
        raise ValueError(f"{name} needs at least {min_len} entries, got {t.numel()}")


def _ptr(t):
    return t.data_ptr() if t is not None and t.numel() > 0 else None


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _common(in_feats, kernel, kpos, in_map, out_map):
    _check_feat("in_feats", in_feats)
    _check_feat("kernel", kernel, in_feats.dtype, dim=3)
    k_vol = kernel.size(0)
    _check_index("kpos", kpos, in_feats.device, k_vol + 1)
    _check_index("in_map", in_map, in_feats.device)
    _check_index("out_map", out_map, in_feats.device)
    if in_map.numel() != out_map.numel():
        raise ValueError("in_map and out_map differ in length")
    return k_vol


_ws_cache: dict = {}


def wgrad_workspace(c_in: int, c_out: int, k_vol: int, device) -> torch.Tensor:
    """fp32 scratch buffer the fp16 weight-gradient needs (cached per device and size)."""
    nbytes = _L.fgms_b200_wgrad_workspace_bytes(c_in, c_out, k_vol, _lib.DTYPE_F16)
    key = (torch.device(device), nbytes)
    ws = _ws_cache.get(key)
    if ws is None:
        ws = torch.empty(max(nbytes // 4, 64), dtype=torch.float32, device=device)
        _ws_cache[key] = ws
    return ws


def fgms_fusion_fwd_cuda(in_feats, kernel, sum_nnz, out_feats, kpos, qkpos, in_map, out_map,
                         separate_mid, arch80):
    """Fused forward — ``ConvolutionForwardFused`` (``backend/spconv.cu:23-246``).

    ``out_feats[out_map[j]] += in_feats[in_map[j]] @ kernel[k(j)]`` for every pair; with
    ``separate_mid`` the centre offset is applied densely and ``out_feats`` is overwritten."""
    k_vol = _common(in_feats, kernel, kpos, in_map, out_map)
    _check_feat("out_feats", out_feats, in_feats.dtype)
    if qkpos is not None:
        _check_index("qkpos", qkpos, in_feats.device, k_vol + 1)
    if out_feats.size(1) != kernel.size(2):
        raise ValueError("out_feats width differs from the kernel's output channels")
    dtype, math = _dtype_math(in_feats, arch80)
    with torch.cuda.device(in_feats.device):
        _lib.check(_L.fgms_b200_fusion_fwd(
            _ptr(in_feats), _ptr(kernel), _ptr(out_feats), _ptr(kpos), _ptr(qkpos), _ptr(in_map), _ptr(out_map),
            in_map.numel(), in_feats.size(0), out_feats.size(0), in_feats.size(1), kernel.size(1), kernel.size(2),
            k_vol, int(sum_nnz), dtype, math, int(bool(separate_mid)), _stream()))


def build_neighbor_table(kpos, in_map, out_map, n_in: int, n_out: int):
    """Neighbour table of the output-stationary forward from the flat pair list: ``nbr[k, r]`` = input row of
    output row ``r`` under offset ``k`` or -1, an int32 tensor ``[k_vol, n_out rounded up to 128]``
    (``fgms_b200_build_neighbor_table``).  Every output row may occur at most once per offset."""
    k_vol = kpos.numel() - 1
    _check_index("kpos", kpos, in_map.device, k_vol + 1)
    _check_index("in_map", in_map, in_map.device, None)
    _check_index("out_map", out_map, in_map.device, in_map.numel())
    nbytes = _L.fgms_b200_neighbor_table_bytes(int(n_out), k_vol)
    nbr = torch.empty((k_vol, nbytes // 4 // k_vol), dtype=torch.int32, device=in_map.device)
    with torch.cuda.device(in_map.device):
        _lib.check(_L.fgms_b200_build_neighbor_table(_ptr(kpos), _ptr(in_map), _ptr(out_map), in_map.numel(), int(n_in),
                                                     int(n_out), k_vol, _ptr(nbr), nbytes, _stream()))
    return nbr


def fgms_fwd_os_cuda(in_feats, kernel, out_feats, nbr, arch80, bias=None, relu=False, accumulate=False):
    """Output-stationary forward (``fgms_b200_fwd_output_stationary``): every output row is computed in one
    accumulator over all offsets and written once — the same bits on every run, with ``bias`` and ReLU applied on
    the way out; ``accumulate=True`` adds to ``out_feats`` as the reference's forward does
    (``backend/spconv.cu:23-246``) and takes neither.  ``nbr`` comes from :func:`build_neighbor_table`.
    Tensor-core shapes only (``ValueError`` otherwise)."""
    _check_feat("in_feats", in_feats, None)
    _check_feat("kernel", kernel, in_feats.dtype, dim=3)
    _check_feat("out_feats", out_feats, in_feats.dtype)
    if kernel.size(1) != in_feats.size(1):
        raise ValueError("Input feature size and kernel size mismatch")
    if out_feats.size(1) != kernel.size(2):
        raise ValueError("out_feats width differs from the kernel's output channels")
    k_vol = kernel.size(0)
    stride = (out_feats.size(0) + 127) // 128 * 128
    if nbr.dtype != torch.int32 or not nbr.is_contiguous() or nbr.device != in_feats.device or nbr.numel() != k_vol * stride:
        raise ValueError("nbr must be the contiguous int32 table build_neighbor_table returns for these sizes")
    if bias is not None:
        _check_feat("bias", bias, in_feats.dtype, dim=1)
        if bias.numel() != kernel.size(2):
            raise ValueError("bias length differs from the kernel's output channels")
    dtype, math = _dtype_math(in_feats, arch80)
    with torch.cuda.device(in_feats.device):
        _lib.check(_L.fgms_b200_fwd_output_stationary(
            _ptr(in_feats), _ptr(kernel), _ptr(out_feats), _ptr(nbr), in_feats.size(0), out_feats.size(0),
            in_feats.size(1), kernel.size(2), k_vol, dtype, math, _ptr(bias), int(bool(relu)), int(bool(accumulate)),
            _stream()))


def fgms_fwd_cuda(in_feats, kernel, sum_nnz, out_feats, kernel_nnz, kernel_pos, in_map, out_map,
                  separate_mid, arch80):
    """Per-offset forward — ``ConvolutionForward`` (``backend/spconv.cu:249-411``).
    ``kernel_nnz`` is a CPU int32 tensor as in the reference (``spconv.cu:308``)."""
    k_vol = _common(in_feats, kernel, kernel_pos, in_map, out_map)
    _check_feat("out_feats", out_feats, in_feats.dtype)
    _check_index("kernel_nnz", kernel_nnz, None, k_vol, cuda=False)
    if out_feats.size(1) != kernel.size(2):
        raise ValueError("out_feats width differs from the kernel's output channels")
    dtype, math = _dtype_math(in_feats, arch80)
    with torch.cuda.device(in_feats.device):
        _lib.check(_L.fgms_b200_seq_fwd(
            _ptr(in_feats), _ptr(kernel), _ptr(out_feats), kernel_nnz.data_ptr(), _ptr(kernel_pos), _ptr(in_map),
            _ptr(out_map), in_map.numel(), in_feats.size(0), out_feats.size(0), in_feats.size(1), kernel.size(1),
            kernel.size(2), k_vol, int(sum_nnz), dtype, math, int(bool(separate_mid)), _stream()))


def fgms_bwd_cuda(out_feats_grad, in_feats, kernel, sum_nnz, in_feats_grad, kernel_grad, kpos, qkpos,
                  in_map, out_map, separate_mid, arch80):
    """Backward — ``ConvolutionBackward`` (``backend/spconv.cu:414-571``): accumulates the input
    gradient into ``in_feats_grad`` and the weight gradient into ``kernel_grad``."""
    k_vol = _common(in_feats, kernel, kpos, in_map, out_map)
    _check_feat("out_feats_grad", out_feats_grad, in_feats.dtype)
    _check_feat("in_feats_grad", in_feats_grad, in_feats.dtype)
    _check_feat("kernel_grad", kernel_grad, in_feats.dtype, dim=3)
    if in_feats.size(1) == kernel.size(1):
        if in_feats_grad.shape != in_feats.shape or kernel_grad.shape != kernel.shape:
            raise ValueError("gradient buffers must have the shapes of in_feats and kernel")
        if out_feats_grad.size(1) != kernel.size(2):
            raise ValueError("out_feats_grad width differs from the kernel's output channels")
    dtype, math = _dtype_math(in_feats, arch80)
    ws = None
    if dtype == _lib.DTYPE_F16 and not _single_launch_wgrad(kernel.size(1), kernel.size(2), k_vol, in_feats.dtype, arch80, None):
        ws = wgrad_workspace(kernel.size(1), kernel.size(2), k_vol, in_feats.device)
    with torch.cuda.device(in_feats.device):
        _lib.check(_L.fgms_b200_bwd(
            _ptr(out_feats_grad), _ptr(in_feats), _ptr(kernel), _ptr(in_feats_grad), _ptr(kernel_grad), _ptr(kpos),
            _ptr(qkpos), _ptr(in_map), _ptr(out_map), in_map.numel(), in_feats.size(0), out_feats_grad.size(0),
            in_feats.size(1), kernel.size(1), kernel.size(2), k_vol, int(sum_nnz), dtype, math, int(bool(separate_mid)),
            _ptr(ws), ws.numel() * 4 if ws is not None else 0, _stream()))


def fgms_dgrad_cuda(out_feats_grad, kernel, in_feats_grad, kpos, in_map, out_map, arch80):
    """Input gradient alone (first half of ``ConvolutionBackward``, ``backend/spconv.cu:454-461``)."""
    k_vol = _common(in_feats_grad, kernel, kpos, in_map, out_map)
    _check_feat("out_feats_grad", out_feats_grad, kernel.dtype)
    dtype, math = _dtype_math(kernel, arch80)
    with torch.cuda.device(kernel.device):
        _lib.check(_L.fgms_b200_dgrad(
            _ptr(out_feats_grad), _ptr(kernel), _ptr(in_feats_grad), _ptr(kpos), _ptr(in_map), _ptr(out_map),
            in_map.numel(), in_feats_grad.size(0), out_feats_grad.size(0), kernel.size(1), kernel.size(2), k_vol,
            dtype, math, _stream()))


# fp16 weight gradients: False = single launch, every CTA adds its fp32 partial sums (rounded to fp16) into
# ``kernel_grad`` with fp16 atomics; True = fp32 sums in a workspace, added to ``kernel_grad`` once at the
# end (three launches).  ``fgms_bwd_cuda`` keeps the reference's signature and follows this switch.
WGRAD_FP32_SUMS = False


def _single_launch_wgrad(c_in, c_out, k_vol, dtype, arch80, fp32_sums) -> bool:
    want_fp32 = WGRAD_FP32_SUMS if fp32_sums is None else fp32_sums
    return dtype == torch.float16 and not want_fp32 and kernel_family("wgrad", c_in, c_out, dtype, arch80, k_vol) == "tcgen05"


def fgms_wgrad_cuda(in_feats, out_feats_grad, kernel_grad, kpos, in_map, out_map, arch80,
                    workspace=None, accumulate=True, fp32_sums=None):
    """Weight gradient alone (second half of ``ConvolutionBackward``, ``backend/spconv.cu:495-569``).

    fp16 storage: with ``accumulate`` and without ``fp32_sums`` (default: ``WGRAD_FP32_SUMS``) and without
    a ``workspace`` the single-launch form runs and ``None`` is returned; otherwise the fp32 sums of this
    call are left in ``workspace`` (returned), which is what a data-parallel caller all-reduces."""
    k_vol = kernel_grad.size(0)
    _check_feat("in_feats", in_feats)
    _check_feat("out_feats_grad", out_feats_grad, in_feats.dtype)
    _check_feat("kernel_grad", kernel_grad, in_feats.dtype, dim=3)
    _check_index("kpos", kpos, in_feats.device, k_vol + 1)
    _check_index("in_map", in_map, in_feats.device)
    _check_index("out_map", out_map, in_feats.device)
    if in_map.numel() != out_map.numel():
        raise ValueError("in_map and out_map differ in length")
    dtype, math = _dtype_math(in_feats, arch80)
    single = workspace is None and accumulate and _single_launch_wgrad(kernel_grad.size(1), kernel_grad.size(2), k_vol,
                                                                       in_feats.dtype, arch80, fp32_sums)
    if dtype == _lib.DTYPE_F16 and workspace is None and not single:
        workspace = wgrad_workspace(kernel_grad.size(1), kernel_grad.size(2), k_vol, in_feats.device)
    with torch.cuda.device(in_feats.device):
        _lib.check(_L.fgms_b200_wgrad(
            _ptr(in_feats), _ptr(out_feats_grad), _ptr(kernel_grad), _ptr(kpos), _ptr(in_map), _ptr(out_map),
            in_map.numel(), in_feats.size(0), out_feats_grad.size(0), kernel_grad.size(1), kernel_grad.size(2), k_vol,
            dtype, math, _ptr(workspace), workspace.numel() * 4 if workspace is not None else 0, int(bool(accumulate)),
            _stream()))
    return workspace


NOALLOC_MAX_ELEMS = 512 * 1024  # FGMS_NOALLOC_MAX_ELEMS in include/fgms_b200.h


def fgms_wgrad_noalloc_cuda(in_feats, out_feats_grad, kernel_grad, kpos, in_map, out_map, arch80=True):
    """fp16 weight gradient through the allocation-free entry point of the library.

    For callers that must not (or cannot) allocate device memory when they call — a serving thread
    where ``cudaMalloc`` is off limits, a process whose memory pool is fully handed out, a thin
    binding with no allocator.  Same result as ``fgms_wgrad_cuda``; the fp32 partial sums use a
    fixed 2 MiB array inside the library, so ``k_vol * c_in * c_out`` may not exceed
    ``NOALLOC_MAX_ELEMS`` (``ValueError`` otherwise).  Calls on one device share that array: do not
    let two of them overlap on the GPU, and make the first call on a device outside stream capture."""
    k_vol = kernel_grad.size(0)
    _check_feat("in_feats", in_feats, torch.float16)
    _check_feat("out_feats_grad", out_feats_grad, torch.float16)
    _check_feat("kernel_grad", kernel_grad, torch.float16, dim=3)
    _check_index("kpos", kpos, in_feats.device, k_vol + 1)
    _check_index("in_map", in_map, in_feats.device)
    _check_index("out_map", out_map, in_feats.device)
    if in_map.numel() != out_map.numel():
        raise ValueError("in_map and out_map differ in length")
    _, math = _dtype_math(in_feats, arch80)
    with torch.cuda.device(in_feats.device):
        _lib.check(_L.fgms_b200_wgrad_f16_noalloc(
            _ptr(in_feats), _ptr(out_feats_grad), _ptr(kernel_grad), _ptr(kpos), _ptr(in_map), _ptr(out_map),
            in_map.numel(), in_feats.size(0), out_feats_grad.size(0), kernel_grad.size(1), kernel_grad.size(2), k_vol,
            math, _stream()))


def wgrad_finalize(kernel_grad: torch.Tensor, partial_f32: torch.Tensor) -> None:
    """``kernel_grad (fp16) += partial_f32`` — the last step of the fp16 weight gradient, exposed so
    that a multi-GPU caller can all-reduce the fp32 partial sums first."""
    _check_feat("kernel_grad", kernel_grad, torch.float16, dim=3)
    if partial_f32.dtype != torch.float32 or not partial_f32.is_cuda or not partial_f32.is_contiguous():
        raise ValueError("partial sums must be a contiguous CUDA float32 tensor")
    if partial_f32.numel() < kernel_grad.numel():
        raise ValueError("partial sums are shorter than kernel_grad")
    with torch.cuda.device(kernel_grad.device):
        _lib.check(_L.fgms_b200_wgrad_finalize(_ptr(kernel_grad), _ptr(partial_f32), kernel_grad.numel(), _stream()))


def kernel_family(pass_: str, c_in: int, c_out: int, dtype: torch.dtype, arch80: bool = True, k_vol: int = 27) -> str:
    """``"tcgen05"`` or ``"simt"``: which kernel family the dispatch uses for a shape (channel counts that are
    multiples of 16 up to 256 whose operands fit shared memory run on tcgen05 unless ``arch80`` is false for
    fp32 storage)."""
    d = _lib.DTYPE_F16 if dtype == torch.float16 else _lib.DTYPE_F32
    m = _lib.MATH_F16 if dtype == torch.float16 else (_lib.MATH_TF32 if arch80 else _lib.MATH_FP32)
    fam = _L.fgms_b200_kernel_family({"fwd": 0, "dgrad": 1, "wgrad": 2}[pass_], c_in, c_out, k_vol, d, m)
    if fam < 0:
        _lib.check(fam)
    return "tcgen05" if fam == 1 else "simt"


def fallback_count() -> int:
    """Launches that should have run on tcgen05 by their shape but ran on the CUDA-core kernels because a
    tensor was not 16-byte aligned (0 in a healthy run)."""
    return int(_L.fgms_b200_fallback_count())


def device_status(reset: bool = True) -> int:
    """Problems kernels reported since the last reset (skipped out-of-range map entries, waits
    that ran out).  Synchronises the current device."""
    v = _L.fgms_b200_device_status(int(reset))
    if v < 0:
        _lib.check(int(v))
    return int(v)


def launch_count() -> int:
    return int(_L.fgms_b200_launch_count())
