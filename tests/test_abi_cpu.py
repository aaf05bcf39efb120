"""CPU-only checks of the boundary: the library builds/loads, exports what include/vafa.h
declares, its struct layout matches the ctypes mirror, and argument errors are reported
without touching a GPU."""
import ctypes as C
import os
import re

import pytest
import torch

from varlenabsorbflashattn_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "vafa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vafa_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.EXPORTS)


def test_abi_version(lib):
    assert lib.vafa_abi_version() == 3


def test_struct_sizes_match_header():
    # 11 pointers + 7 int32 + float + 3 int32 (+pad) + pointer + size_t + pointer + num_kv_heads (int32, padded to 8)
    assert C.sizeof(_lib.VarlenArgs) == 11 * 8 + 12 * 4 + 3 * 8 + 8
    # ... + x_width (int32, padded to 8)
    assert C.sizeof(_lib.AbsorbArgs) == 14 * 8 + 12 * 4 + 3 * 8 + 8


def test_null_args_rejected(lib):
    assert lib.vafa_varlen_fwd(None, None) == -1
    assert b"null" in lib.vafa_last_error()


def test_bad_head_dim_rejected(lib):
    a = _lib.VarlenArgs()
    a.n_seg, a.total_q, a.total_k, a.num_heads, a.head_dim, a.dtype = 1, 0, 0, 1, 48, 1
    assert lib.vafa_varlen_fwd(C.byref(a), None) == -2
    assert b"head_dim" in lib.vafa_last_error()


def test_bad_split_rejected(lib):
    a = _lib.VarlenArgs()
    a.n_seg, a.total_q, a.total_k, a.num_heads, a.head_dim, a.dtype = 1, 0, 0, 1, 64, 1
    cu = (C.c_int32 * 2)(0, 0)
    a.cu_seqlens_q = a.cu_seqlens_k = C.cast(cu, C.c_void_p)
    a.split_k_block = 100
    assert lib.vafa_varlen_fwd(C.byref(a), None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_absorb_narrow_x_needs_a_valid_width(lib):
    """x_width (rows of x / dx narrower than d_kv) must be a multiple of 8 and at most d_kv; the check runs
    before anything touches the device."""
    a = _lib.AbsorbArgs()
    a.n_seg, a.total_q, a.total_k, a.num_heads, a.head_dim, a.dtype = 1, 0, 0, 8, 32, 1
    a.d_q, a.d_kv = 256, 256
    cu = (C.c_int32 * 2)(0, 0)
    a.cu_seqlens_q = a.cu_seqlens_k = C.cast(cu, C.c_void_p)
    dummy = (C.c_char * 64)()
    a.w_q = a.w_k = a.w_v = C.cast(dummy, C.c_void_p)
    a.x_width = 300
    assert lib.vafa_absorb_fwd(C.byref(a), None) == -1
    assert b"x_width" in lib.vafa_last_error()
    a.x_width = 212
    assert lib.vafa_absorb_fwd(C.byref(a), None) == -1
    # a valid narrow width without the tensor-core path (nothing to attend over here) is refused as unsupported
    a.x_width = 216
    assert lib.vafa_absorb_fwd(C.byref(a), None) == -2
    assert b"tcgen05" in lib.vafa_last_error()


def test_kv_head_count_must_divide_the_query_heads(lib):
    a = _lib.VarlenArgs()
    a.n_seg, a.total_q, a.total_k, a.num_heads, a.head_dim, a.dtype = 1, 0, 0, 6, 64, 1
    cu = (C.c_int32 * 2)(0, 0)
    a.cu_seqlens_q = a.cu_seqlens_k = C.cast(cu, C.c_void_p)
    a.num_kv_heads = 4
    assert lib.vafa_varlen_fwd(C.byref(a), None) == -1
    assert b"num_kv_heads" in lib.vafa_last_error()
