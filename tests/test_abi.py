"""The C-ABI library builds, loads and exports what include/sa2.h declares.
No kernel is launched here (these run without a GPU)."""
import ctypes as C
import os
import re

import pytest

from simplicial_attention_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "sa2.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sa2_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = _lib.lib()
    names = _declared()
    assert set(_lib.EXPORTS) <= set(names)
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/sa2.h but not exported"


def test_struct_layout_matches_header():
    # 12 x int32/float in sa2_shape; pointers and strides are 8-byte fields
    assert C.sizeof(_lib.Shape) == 48
    assert C.sizeof(_lib.Strides) == 24
    assert C.sizeof(_lib.FwdArgs) == 48 + 7 * 8 + 6 * 24 + 8
    assert C.sizeof(_lib.BwdArgs) == 48 + 13 * 8 + 12 * 24 + 8 + 8 + 8 + 8


def test_status_strings_and_version():
    lib = _lib.lib()
    assert lib.sa2_version() >= 100
    for code in range(6):
        assert lib.sa2_strerror(code)
    assert b"unknown" in lib.sa2_strerror(99)


def _shape(**kw):
    base = dict(b=1, n=64, hq=2, hk=2, d=64, w1=16, w2=4, off1=0, off2=0, dtype=0, kernel=0, scale=0.125)
    base.update(kw)
    return _lib.Shape(*[base[f[0]] for f in _lib.Shape._fields_])


def test_argument_errors_are_status_codes_not_crashes():
    lib = _lib.lib()
    assert lib.sa2_fwd(None) == 1
    assert lib.sa2_bwd(None) == 1
    a = _lib.FwdArgs()
    a.shape = _shape(d=48)
    assert lib.sa2_fwd(C.byref(a)) == 2          # unsupported head dim
    a.shape = _shape(hq=3, hk=2)
    assert lib.sa2_fwd(C.byref(a)) == 1          # heads not divisible
    a.shape = _shape()
    assert lib.sa2_fwd(C.byref(a)) == 1          # null pointers
    a.shape = _shape(dtype=7)
    assert lib.sa2_fwd(C.byref(a)) == 2
    b = _lib.BwdArgs()
    b.shape = _shape()
    assert lib.sa2_bwd(C.byref(b)) == 1


def test_workspace_size():
    lib = _lib.lib()
    s = _shape(b=2, n=100, hq=4, hk=2)
    need = lib.sa2_bwd_workspace_bytes(C.byref(s))
    assert need >= 2 * 4 * 100 * 4 and need % 256 == 0
    assert lib.sa2_bwd_workspace_bytes(C.byref(_shape(d=48))) == 0


def test_headnorm_argument_errors():
    lib = _lib.lib()
    assert lib.sa2_headnorm_fwd(None) == 1 and lib.sa2_headnorm_bwd(None) == 1
    a = _lib.HeadnormArgs()
    assert lib.sa2_headnorm_fwd(C.byref(a)) == 1                     # null pointers
    # fake (never dereferenced) addresses: validation happens before any launch
    a.x, a.weight, a.y, a.rstd = 256, 256, 256, 256
    a.rows, a.channels, a.x_stride, a.y_stride = 8, 96, 96, 96
    a.d = 48
    assert lib.sa2_headnorm_fwd(C.byref(a)) == 2                     # group width not supported
    a.d, a.channels = 64, 96
    assert lib.sa2_headnorm_fwd(C.byref(a)) == 1                     # channels not a multiple of d
    a.channels, a.x_stride, a.y_stride = 128, 128, 100
    assert lib.sa2_headnorm_fwd(C.byref(a)) == 1                     # row stride shorter than a row
    a.y_stride, a.x_dtype = 128, 9
    assert lib.sa2_headnorm_fwd(C.byref(a)) == 2                     # unknown dtype
    a.x_dtype = 0
    a.dy, a.dweight, a.dy_stride = 256, 256, 128
    assert lib.sa2_headnorm_bwd(C.byref(a)) == 3                     # scratch missing
    assert lib.sa2_headnorm_partial_bytes(8, 128) == 1 * 128 * 4
    assert lib.sa2_headnorm_partial_bytes(10 ** 6, 1536) == 592 * 1536 * 4
    assert lib.sa2_headnorm_partial_bytes(0, 128) == 0
