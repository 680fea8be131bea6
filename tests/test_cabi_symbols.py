"""The shared library loads and exports every entry point that include/*.h declares
(no kernel is launched here: this runs without a GPU)."""

import ctypes
import re

import pytest

from conftest import ROOT


def declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(bt_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def built_lib():
    from bastile_b200 import build

    return ctypes.CDLL(str(build.build()))


def test_header_declares_something():
    assert len(declared_symbols()) >= 10


@pytest.mark.parametrize("name", declared_symbols())
def test_symbol_is_exported(built_lib, name):
    assert getattr(built_lib, name) is not None


def test_python_binding_covers_the_header():
    from bastile_b200._lib import SIGNATURES

    assert sorted(SIGNATURES) == declared_symbols()


def test_version_and_error_text_without_gpu(built_lib):
    built_lib.bt_version.restype = ctypes.c_int
    built_lib.bt_last_error.restype = ctypes.c_char_p
    assert built_lib.bt_version() >= 100
    assert isinstance(built_lib.bt_last_error(), bytes)


def test_argument_errors_are_reported_not_thrown():
    """Shape validation happens on the host before any launch, so it can be checked here."""
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    rc = lib.bt_rmsnorm_fwd(None, None, None, None, 4, 0, 0, 0, 1e-6, _lib.BT_BF16, None)
    assert rc == -1 and b"rmsnorm_fwd" in lib.bt_last_error()
    s3 = _lib.I64x3(0, 0, 0)
    rc = lib.bt_rope(None, None, None, None, None, None, 1, 1, 1, 1, 63, s3, s3, s3, s3, _lib.I64x2(0, 0), 1, 0,
                     _lib.BT_BF16, None)
    assert rc == -1 and b"head_dim" in lib.bt_last_error()


def test_argument_errors_of_the_fused_entry_points():
    """Host-side validation of the entry points added for the fused decoder-layer path."""
    import ctypes as C

    from bastile_b200 import _lib

    lib = _lib.get_lib()
    one = C.c_void_p(16)  # never dereferenced: validation fails before any launch
    rc = lib.bt_add_rmsnorm_fwd(one, one, one, one, one, one, 4, 128, 64, 128, 128, 128, 1e-6, _lib.BT_BF16, None)
    assert rc == -1 and b"row stride" in lib.bt_last_error()
    rc = lib.bt_add_rmsnorm_fwd(one, one, one, one, one, one, 4, 128, 128, 128, 128, 128, 1e-6, _lib.BT_BF16, None)
    assert rc == -1 and b"alias" in lib.bt_last_error()
    rc = lib.bt_add_rmsnorm_bwd(one, one, one, one, None, one, one, one, 4, 128, 128, 128, 128, 128, _lib.BT_BF16, None)
    assert rc == -1 and b"null pointer" in lib.bt_last_error()
    s3, s2 = _lib.I64x3(0, 0, 0), _lib.I64x2(0, 0)
    rc = lib.bt_qk_norm_rope_fwd(one, one, one, one, one, one, one, one, one, one, 1, 4, 2, 0, 128, s3, s3, s3, s3, s2,
                                 1, 1e-6, 1e-6, _lib.BT_BF16, None)
    assert rc == -1 and b"at least one head" in lib.bt_last_error()
    rc = lib.bt_qk_norm_rope_fwd(one, one, one, one, one, one, one, one, one, one, 2, 4, 2, 2, 128, s3, s3, s3, s3, s2,
                                 3, 1e-6, 1e-6, _lib.BT_BF16, None)
    assert rc == -1 and b"cos batch" in lib.bt_last_error()
    assert lib.bt_gemm_ex(None, None, None) == -1 and b"null descriptor" in lib.bt_last_error()
    d = _lib.GemmDesc()
    d.A = d.B = d.D = 16
    d.M, d.N, d.K, d.lda, d.ldb, d.ldd = 8, 8, 8, 8, 8, 8
    d.in_dtype, d.out_dtype = _lib.BT_BF16, _lib.BT_FP16
    assert lib.bt_gemm_ex(C.byref(d), None, None) == -1 and b"result must have" in lib.bt_last_error()
    d.out_dtype = _lib.BT_BF16
    d.A1 = 16  # a second product without its B
    assert lib.bt_gemm_ex(C.byref(d), None, None) == -1 and b"no B1" in lib.bt_last_error()
    arr = (C.c_void_p * 1)(16)
    n = (C.c_int64 * 1)(8)
    rc = lib.bt_adamw_step(arr, arr, arr, arr, n, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, 99, _lib.BT_BF16, None)
    assert rc == -1 and b"ctas_per_sm" in lib.bt_last_error()
    assert lib.bt_set_gemm_dynamic_tiles(-1) in (0, 1)
