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
