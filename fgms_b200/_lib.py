"""ctypes view of ``libfgms_b200.so`` (the C ABI declared in ``include/fgms_b200.h``).

There is no fallback of any kind: if the shared library is missing or a symbol cannot be
resolved, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfgms_b200.so")

OK = 0
ERR_INVALID_ARG, ERR_CHANNEL_MISMATCH, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE = -1, -2, -3, -4, -5, -6
DTYPE_F32, DTYPE_F16 = 0, 1
MATH_FP32, MATH_TF32, MATH_F16 = 0, 1, 2

# name -> (restype, argtypes); mirrors include/fgms_b200.h declaration by declaration
SIGNATURES = {
    "fgms_b200_fusion_fwd": (c_int, [c_void_p] * 7 + [c_int64] + [c_int] * 6 + [c_int64] + [c_int] * 3 + [c_void_p]),
    "fgms_b200_seq_fwd": (c_int, [c_void_p] * 7 + [c_int64] + [c_int] * 6 + [c_int64] + [c_int] * 3 + [c_void_p]),
    "fgms_b200_dgrad": (c_int, [c_void_p] * 6 + [c_int64] + [c_int] * 7 + [c_void_p]),
    "fgms_b200_wgrad": (c_int, [c_void_p] * 6 + [c_int64] + [c_int] * 7 + [c_void_p, c_size_t, c_int, c_void_p]),
    "fgms_b200_wgrad_finalize": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "fgms_b200_wgrad_f16_noalloc": (c_int, [c_void_p] * 6 + [c_int64] + [c_int] * 6 + [c_void_p]),
    "fgms_b200_wgrad_workspace_bytes": (c_size_t, [c_int] * 4),
    "fgms_b200_bwd": (c_int, [c_void_p] * 9 + [c_int64] + [c_int] * 6 + [c_int64] + [c_int] * 3 + [c_void_p, c_size_t, c_void_p]),
    "fgms_b200_map_workspace_bytes": (c_size_t, [c_int] * 3),
    "fgms_b200_build_submanifold_map": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                                c_void_p, c_void_p]),
    "fgms_b200_build_strided_map": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_size_t, c_void_p, c_void_p]),
    "fgms_b200_transpose_map": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_size_t, c_void_p]),
    "fgms_b200_neighbor_table_bytes": (c_size_t, [c_int, c_int]),
    "fgms_b200_build_neighbor_table": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "fgms_b200_fwd_output_stationary": (c_int, [c_void_p] * 4 + [c_int] * 7 + [c_void_p, c_int, c_int, c_void_p]),
    "fgms_b200_peer_exchange_flag_bytes": (c_size_t, [c_int]),
    "fgms_b200_peer_exchange": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, ctypes.c_uint32, c_int64, c_int, c_void_p]),
    "fgms_b200_kernel_family": (c_int, [c_int] * 6),
    "fgms_b200_fallback_count": (c_int64, []),
    "fgms_b200_set_reserved_sms": (c_int, [c_int]),
    "fgms_b200_device_status": (c_int64, [c_int]),
    "fgms_b200_launch_count": (c_int64, []),
    "fgms_b200_last_error": (c_char_p, []),
    "fgms_b200_version": (c_char_p, []),
}


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m fgms_b200.build` "
            "(nvcc, sm_100a). fgms_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    return lib.fgms_b200_last_error().decode()


def check(rc: int) -> None:
    """Turn a C-ABI status into the exception the reference binding would raise."""
    if rc == OK:
        return
    msg = last_error()
    if rc in (ERR_CHANNEL_MISMATCH, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE):
        raise ValueError(msg)  # pybind11 maps std::invalid_argument to ValueError
    raise RuntimeError(f"fgms_b200 error {rc}: {msg}")
