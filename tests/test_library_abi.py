"""CPU-side checks of the C ABI: the library loads and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from cudf_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b2_groupby.h")


def declared_symbols():
    text = open(HEADER, encoding="utf-8").read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_loads():
    path = build.build()
    assert os.path.exists(path)
    lib = _lib.load()
    assert b"sm_100a" in lib.b2_version()


def test_every_declared_symbol_is_exported():
    lib = ctypes.CDLL(build.build())
    names = declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/b2_groupby.h but not exported"


def test_binding_covers_the_header():
    assert sorted(_lib.PROTOTYPES) == declared_symbols()


def test_struct_sizes_match_the_header():
    # natural alignment on LP64; a mismatch here would corrupt every call
    assert ctypes.sizeof(_lib.ColumnView) == 48
    assert ctypes.sizeof(_lib.Aggregation) == 8
    assert ctypes.sizeof(_lib.AggregationRequest) == 64
    assert ctypes.sizeof(_lib.OwnedColumn) == 64
    assert ctypes.sizeof(_lib.Allocator) == 24
    assert ctypes.sizeof(_lib.GroupbyOptions) == 40
    assert ctypes.sizeof(_lib.CallStats) == 32


def test_argument_errors_need_no_gpu():
    lib = _lib.load()
    out = ctypes.c_void_p()
    assert lib.b2_groupby_create(None, 1, 0, None, ctypes.byref(out)) == _lib.Status.INVALID_ARGUMENT
    assert b"keys is null" in lib.b2_last_error()
    v = (_lib.ColumnView * 1)()
    v[0].type_id, v[0].size = 3, 0
    assert lib.b2_groupby_create(v, 1, 7, None, ctypes.byref(out)) == _lib.Status.INVALID_ARGUMENT
    # finishers over partial columns: what is wrong with the arguments is said before anything touches a GPU
    oc = _lib.OwnedColumn()
    assert lib.b2_finish_partial(10, 1, 10, None, None, None, 0, None, None, ctypes.byref(oc)) == _lib.Status.INVALID_ARGUMENT
    cnt = (_lib.ColumnView * 1)()
    cnt[0].type_id, cnt[0].size = 4, 5        # INT64 counts
    assert lib.b2_finish_partial(99, 1, 10, None, cnt, None, 0, None, None, ctypes.byref(oc)) == _lib.Status.INVALID_ARGUMENT
    assert lib.b2_finish_partial(10, 1, 10, None, cnt, None, 0, None, None, ctypes.byref(oc)) == _lib.Status.INVALID_ARGUMENT   # MEAN
    assert b"sum column is missing" in lib.b2_last_error()
    cnt[0].type_id = 10                       # FLOAT64 is not a count
    assert lib.b2_finish_partial(5, 1, 3, None, cnt, None, 0, None, None, ctypes.byref(oc)) == _lib.Status.DATA_TYPE_ERROR      # COUNT_VALID


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.LibraryMissing, match="no CPU fallback"):
        _lib.load()


def test_comm_entry_points_reject_bad_arguments():
    """The multi-GPU entry points (no GPU needed for the argument checks)."""
    lib = _lib.load()
    handle = ctypes.c_void_p()
    ident = (ctypes.c_uint8 * 128)()
    assert lib.b2_comm_create(ident, 2, 2, ctypes.byref(handle)) == _lib.Status.INVALID_ARGUMENT
    assert lib.b2_comm_create(None, 0, 1, ctypes.byref(handle)) == _lib.Status.INVALID_ARGUMENT
    assert lib.b2_comm_adopt(None, 0, 1, ctypes.byref(handle)) == _lib.Status.INVALID_ARGUMENT
    assert handle.value is None
    assert lib.b2_groupby_aggregate_multi(None, None, None, 0, None, None, None) == _lib.Status.INVALID_ARGUMENT
    lib.b2_comm_destroy(None)
