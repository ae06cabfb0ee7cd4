"""The C-ABI library: it loads, exports every symbol the header declares, and rejects bad
arguments before touching a device (these checks run without a GPU)."""
import ctypes
import os
import re

import pytest

from fgms_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(fgms_b200_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    declared = _declared_symbols()
    assert len(declared) >= 10
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), f"{name} is declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes signatures out of step with the header"
    assert b"sm_100a" in _lib.lib.fgms_b200_version()


def test_channel_mismatch_is_the_reference_error():
    L = _lib.lib
    rc = L.fgms_b200_fusion_fwd(None, None, None, None, None, None, None, 0, 4, 4, 16, 8, 16, 27, 0, 0, 0, 0, None)
    assert rc == _lib.ERR_CHANNEL_MISMATCH
    assert _lib.last_error() == "Input feature size and kernel size mismatch"  # backend/spconv.cu:39-43
    with pytest.raises(ValueError, match="Input feature size and kernel size mismatch"):
        _lib.check(rc)
    rc = L.fgms_b200_bwd(None, None, None, None, None, None, None, None, None, 0, 4, 4, 16, 8, 16, 27, 0, 0, 0, 0, None, 0, None)
    assert rc == _lib.ERR_CHANNEL_MISMATCH


@pytest.mark.parametrize("args,code", [
    (dict(dtype=7), _lib.ERR_INVALID_ARG),
    (dict(math=9), _lib.ERR_INVALID_ARG),
    (dict(dtype=_lib.DTYPE_F16, math=_lib.MATH_TF32), _lib.ERR_UNSUPPORTED),
    (dict(dtype=_lib.DTYPE_F32, math=_lib.MATH_F16), _lib.ERR_UNSUPPORTED),
    (dict(k_vol=0), _lib.ERR_INVALID_ARG),
    (dict(c_out=0), _lib.ERR_INVALID_ARG),
    (dict(n_in=-1), _lib.ERR_INVALID_ARG),
    (dict(sum_nnz=-5), _lib.ERR_INVALID_ARG),
    (dict(separate_mid=1, n_out=5), _lib.ERR_INVALID_ARG),
    (dict(map_len=-1), _lib.ERR_INVALID_ARG),
    (dict(map_len=2 ** 31), _lib.ERR_INVALID_ARG),
    (dict(), _lib.ERR_INVALID_ARG),  # null kernel / kpos
])
def test_argument_validation_without_a_device(args, code):
    a = dict(n_in=4, n_out=4, c_in=8, c_out=8, k_vol=27, sum_nnz=0, dtype=0, math=0, separate_mid=0, map_len=0)
    a.update(args)
    rc = _lib.lib.fgms_b200_fusion_fwd(None, None, None, None, None, None, None, a["map_len"], a["n_in"], a["n_out"],
                                       a["c_in"], a["c_in"], a["c_out"], a["k_vol"], a["sum_nnz"], a["dtype"], a["math"],
                                       a["separate_mid"], None)
    assert rc == code, _lib.last_error()
    assert _lib.last_error()


def test_workspace_size_and_family_queries():
    L = _lib.lib
    assert L.fgms_b200_wgrad_workspace_bytes(128, 128, 27, _lib.DTYPE_F16) == 27 * 128 * 128 * 4
    assert L.fgms_b200_wgrad_workspace_bytes(128, 128, 27, _lib.DTYPE_F32) == 0
    assert L.fgms_b200_kernel_family(0, 16, 16, 27, _lib.DTYPE_F32, _lib.MATH_FP32) == 0
    assert L.fgms_b200_kernel_family(0, 128, 128, 27, _lib.DTYPE_F32, _lib.MATH_FP32) == 0  # fp32 math is never tensor-core
    assert L.fgms_b200_kernel_family(0, 17, 33, 27, _lib.DTYPE_F16, _lib.MATH_F16) == 0
    assert L.fgms_b200_launch_count() >= 0 and L.fgms_b200_fallback_count() == 0
    # tensor-core shapes: channel counts that are multiples of 16, at most 256, whose operands fit shared memory
    F16, F32, M16, TF = _lib.DTYPE_F16, _lib.DTYPE_F32, _lib.MATH_F16, _lib.MATH_TF32
    fam = lambda ci, co, dt, m, kv=27: [L.fgms_b200_kernel_family(ps, ci, co, kv, dt, m) for ps in range(3)]
    assert fam(128, 128, F16, M16) == [1, 1, 1]
    assert fam(256, 256, F16, M16) == [1, 1, 1]
    assert fam(64, 192, F16, M16) == [1, 1, 1]
    assert fam(192, 64, F16, M16) == [1, 1, 1]      # 192 gradient rows: a 128-row and a 64-row tile
    assert fam(96, 32, F32, TF) == [1, 1, 1]
    assert fam(32, 64, F32, TF, 8) == [1, 1, 1]
    assert fam(32, 32, F16, M16) == [1, 1, 1]       # 64-byte rows
    assert fam(16, 16, F16, M16) == [1, 1, 1]       # 32-byte rows
    assert fam(48, 80, F16, M16) == [1, 1, 1]
    assert fam(4, 32, F16, M16) == [0, 0, 0]        # not a multiple of 16
    assert fam(24, 32, F32, TF) == [0, 0, 0]
    assert fam(320, 64, F16, M16) == [0, 0, 0]      # more than 256 channels
    assert fam(256, 256, F32, TF) == [0, 0, 1]      # a 256 KB tf32 weight matrix does not fit shared memory
    assert fam(128, 128, F16, M16, 4096)[0] in (0, 1)  # a large k_vol only grows the tile table
    assert L.fgms_b200_kernel_family(3, 64, 64, 27, F16, M16) < 0
    assert L.fgms_b200_kernel_family(0, 64, 64, 0, F16, M16) < 0
    # map-builder workspace: grows with both the table and the dense [k_vol x columns] scratch
    w = L.fgms_b200_map_workspace_bytes
    assert w(0, 0, 27) > 0 and w(1000, 1000, 27) < w(2000, 1000, 27) < w(2000, 2000, 27) and w(1000, 1000, 27) % 256 == 0
    assert w(-1, 10, 27) == 0 and w(10, 10, 0) == 0


def test_map_builders_validate_without_a_device():
    L = _lib.lib
    assert L.fgms_b200_build_submanifold_map(None, 10, 4, None, None, None, None, 0, None, None) == _lib.ERR_INVALID_ARG  # even kernel
    assert L.fgms_b200_build_submanifold_map(None, -1, 3, None, None, None, None, 0, None, None) == _lib.ERR_INVALID_ARG
    assert L.fgms_b200_build_strided_map(None, 10, 1, None, None, None, None, None, 0, None, None) == _lib.ERR_INVALID_ARG  # stride < 2
    assert L.fgms_b200_transpose_map(None, None, None, 5, 0, 0, None, None, None, None, 0, None) == _lib.ERR_INVALID_ARG
    assert _lib.last_error()


def test_seq_forward_checks_host_counts():
    import numpy as np
    knnz = np.array([1, 2, 3], dtype=np.int32)
    one = ctypes.c_void_p(8)  # never dereferenced: validation fails first
    rc = _lib.lib.fgms_b200_seq_fwd(one, one, one, knnz.ctypes.data, one, one, one, 7, 4, 4, 8, 8, 8, 3, 7, 0, 0, 0, None)
    assert rc == _lib.ERR_INVALID_ARG and "sums to 6" in _lib.last_error()
    rc = _lib.lib.fgms_b200_seq_fwd(one, one, one, knnz.ctypes.data, one, one, one, 5, 4, 4, 8, 8, 8, 3, 6, 0, 0, 0, None)
    assert rc == _lib.ERR_INVALID_ARG and "maps hold 5" in _lib.last_error()


def test_maps_may_be_null_only_when_empty():
    one = ctypes.c_void_p(8)  # never dereferenced: validation fails first
    L = _lib.lib
    rc = L.fgms_b200_dgrad(one, one, one, one, None, one, 3, 4, 4, 8, 8, 27, 0, 0, None)
    assert rc == _lib.ERR_INVALID_ARG and "map pointer" in _lib.last_error()
    rc = L.fgms_b200_wgrad(one, one, one, one, one, None, 3, 4, 4, 8, 8, 27, 0, 0, None, 0, 1, None)
    assert rc == _lib.ERR_INVALID_ARG and "map pointer" in _lib.last_error()
    rc = L.fgms_b200_wgrad_f16_noalloc(one, one, one, one, None, None, 1, 4, 4, 8, 8, 27, 2, None)
    assert rc == _lib.ERR_INVALID_ARG


def test_peer_exchange_validates_without_a_device():
    L = _lib.lib
    assert L.fgms_b200_peer_exchange_flag_bytes(8) >= (2 * 8 + 1) * 4 and L.fgms_b200_peer_exchange_flag_bytes(8) % 256 == 0
    assert L.fgms_b200_peer_exchange_flag_bytes(0) == 0 and L.fgms_b200_peer_exchange_flag_bytes(17) == 0
    tab = (ctypes.c_void_p * 2)(16, 32)  # never dereferenced: validation fails first
    call = lambda rank, world, count, ctas=8: L.fgms_b200_peer_exchange(tab, tab, tab, rank, world, count, 1, 0, ctas, None)
    assert call(0, 0, 16) == _lib.ERR_INVALID_ARG
    assert call(2, 2, 16) == _lib.ERR_INVALID_ARG and "rank" in _lib.last_error()
    assert call(0, 2, 18) == _lib.ERR_INVALID_ARG and "multiple of 4" in _lib.last_error()
    assert call(0, 2, 16, ctas=0) == _lib.ERR_INVALID_ARG
    assert L.fgms_b200_peer_exchange(None, tab, tab, 0, 2, 16, 1, 0, 8, None) == _lib.ERR_INVALID_ARG
    odd = (ctypes.c_void_p * 2)(16, 40)  # rank 1's buffer is not 16-byte aligned
    assert L.fgms_b200_peer_exchange(odd, tab, tab, 0, 2, 16, 1, 0, 8, None) == _lib.ERR_INVALID_ARG


def test_reserved_sm_setting_validates():
    L = _lib.lib
    assert L.fgms_b200_set_reserved_sms(-1) == _lib.ERR_INVALID_ARG
    assert L.fgms_b200_set_reserved_sms(65) == _lib.ERR_INVALID_ARG
    assert L.fgms_b200_set_reserved_sms(8) == _lib.OK
    assert L.fgms_b200_set_reserved_sms(0) == _lib.OK


def test_output_stationary_forward_validates_without_a_device():
    L = _lib.lib
    assert L.fgms_b200_neighbor_table_bytes(0, 27) == 0
    assert L.fgms_b200_neighbor_table_bytes(1, 27) == 27 * 128 * 4
    assert L.fgms_b200_neighbor_table_bytes(146546, 27) == 27 * 146560 * 4
    p = 256  # never dereferenced: validation fails first
    build = lambda kpos, imap, omap, map_len, nbr, nbytes, k_vol=27: L.fgms_b200_build_neighbor_table(
        kpos, imap, omap, map_len, 10, 10, k_vol, nbr, nbytes, None)
    assert build(None, p, p, 4, p, 1 << 20) == _lib.ERR_INVALID_ARG
    assert build(p, None, p, 4, p, 1 << 20) == _lib.ERR_INVALID_ARG
    assert build(p, p, p, 4, p, 16) == _lib.ERR_WORKSPACE
    assert build(p, p, p, 4, p, 1 << 20, k_vol=0) == _lib.ERR_INVALID_ARG
    fwd = lambda dtype, math, bias=None, relu=0, acc=0, c_in=32, nbr=p: L.fgms_b200_fwd_output_stationary(
        p, p, p, nbr, 10, 10, c_in, 32, 27, dtype, math, bias, relu, acc, None)
    assert fwd(_lib.DTYPE_F16, _lib.MATH_TF32) == _lib.ERR_UNSUPPORTED
    assert fwd(_lib.DTYPE_F16, _lib.MATH_F16, bias=p, acc=1) == _lib.ERR_INVALID_ARG and "accumulate" in _lib.last_error()
    assert fwd(_lib.DTYPE_F16, _lib.MATH_F16, relu=1, acc=1) == _lib.ERR_INVALID_ARG
    assert fwd(_lib.DTYPE_F16, _lib.MATH_F16, nbr=None) == _lib.ERR_INVALID_ARG
    assert fwd(_lib.DTYPE_F16, _lib.MATH_F16, c_in=0) == _lib.ERR_INVALID_ARG
