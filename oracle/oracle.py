"""ctypes front end of the CPU oracle (oracle/groupby_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of bench.py as the checker and the timed CPU
baseline.  The shipped package (cudf_b200/) never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import List, Optional, Sequence, Tuple

import numpy as np

from cudf_b200.types import HostColumn, Kind, NullPolicy, STORAGE_DTYPE, TypeId

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class _Col(C.Structure):
    _fields_ = [("type_id", C.c_int32), ("size", C.c_int32), ("data", C.c_void_p),
                ("mask", C.c_void_p), ("offset", C.c_int32), ("offsets_type", C.c_int32),
                ("offsets", C.c_void_p)]


class _Agg(C.Structure):
    _fields_ = [("kind", C.c_int32), ("ddof", C.c_int32)]


class _Req(C.Structure):
    _fields_ = [("values", _Col), ("naggs", C.c_int32), ("aggs", C.POINTER(_Agg))]


def build(force: bool = False) -> str:
    """Compiles liboracle.so with g++ (oracle/Makefile) when missing or stale."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "groupby_oracle.cpp")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def _lib():
    global _LIB
    if _LIB is None:
        lib = C.CDLL(build())
        lib.orc_groupby.restype = C.c_void_p
        lib.orc_groupby.argtypes = [C.POINTER(_Col), C.c_int32, C.c_int32, C.POINTER(_Req), C.c_int32,
                                    C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.c_int32, C.c_int32]
        lib.orc_error.restype = C.c_char_p
        lib.orc_error.argtypes = [C.c_void_p]
        lib.orc_num_groups.restype = C.c_int64
        lib.orc_num_groups.argtypes = [C.c_void_p]
        for name, rt in (("orc_col_type", C.c_int32), ("orc_col_bytes", C.c_int64),
                         ("orc_col_data", C.c_void_p), ("orc_col_mask", C.c_void_p),
                         ("orc_col_null_count", C.c_int64), ("orc_col_offsets", C.c_void_p),
                         ("orc_col_child_type", C.c_int32), ("orc_col_data2", C.c_void_p),
                         ("orc_col_bytes2", C.c_int64)):
            f = getattr(lib, name)
            f.restype = rt
            f.argtypes = [C.c_void_p, C.c_int32, C.c_int32]
        lib.orc_free.argtypes = [C.c_void_p]
        lib.orc_free.restype = None
        _LIB = lib
    return _LIB


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data


def _to_c(col: HostColumn, keep: list) -> _Col:
    data = None if col.data is None else np.ascontiguousarray(col.data)
    mask = None if col.mask is None else np.ascontiguousarray(col.mask, dtype=np.uint32)
    offs = None if col.offsets is None else np.ascontiguousarray(col.offsets)
    keep.extend([data, mask, offs])
    ot = 0
    if offs is not None:
        ot = int(TypeId.INT64 if offs.dtype == np.int64 else TypeId.INT32)
    return _Col(int(col.type_id), int(col.size), _ptr(data), _ptr(mask), int(col.offset), ot, _ptr(offs))


class OracleError(RuntimeError):
    pass


def groupby(keys: Sequence[HostColumn], requests: Sequence[Tuple[HostColumn, Sequence]],
            null_policy: int = NullPolicy.EXCLUDE,
            row_filters: Sequence[np.ndarray] = (), row_filter_offsets: Sequence[int] = (),
            threads: int = 1) -> Tuple[List[HostColumn], List[List[HostColumn]]]:
    """Reference semantics of ``groupby(keys, null_policy).aggregate(requests)`` on the CPU.

    ``requests`` is a list of (values column, [aggregation, ...]) where an aggregation is a kind
    or a (kind, ddof) pair.  Returns (key columns, per-request result columns); group order is the
    order of first appearance (callers sort by key before comparing)."""
    lib = _lib()
    keep: list = []
    ckeys = (_Col * len(keys))(*[_to_c(k, keep) for k in keys])
    creqs = (_Req * max(1, len(requests)))()
    for i, (vals, aggs) in enumerate(requests):
        arr = (_Agg * max(1, len(aggs)))()
        for j, a in enumerate(aggs):
            kind, ddof = (a if isinstance(a, tuple) else (a, 1))
            arr[j] = _Agg(int(kind), int(ddof))
        keep.append(arr)
        creqs[i] = _Req(_to_c(vals, keep), len(aggs), arr)
    nf = len(row_filters)
    fl = [np.ascontiguousarray(f, dtype=np.uint32) for f in row_filters]
    keep.append(fl)
    fptr = (C.c_void_p * max(1, nf))(*[f.ctypes.data for f in fl])
    foff = (C.c_int32 * max(1, nf))(*([int(o) for o in row_filter_offsets] or [0] * nf))
    h = lib.orc_groupby(ckeys, len(keys), int(null_policy), creqs, len(requests), fptr, foff, nf,
                        int(threads))
    try:
        err = lib.orc_error(h)
        if err:
            raise OracleError(err.decode())
        ngroups = lib.orc_num_groups(h)

        def fetch(req: int, idx: int, scale: int = 0) -> HostColumn:
            t = TypeId(lib.orc_col_type(h, req, idx))
            nbytes = lib.orc_col_bytes(h, req, idx)
            raw = np.ctypeslib.as_array((C.c_uint8 * nbytes).from_address(lib.orc_col_data(h, req, idx))).copy() \
                if nbytes else np.zeros(0, np.uint8)
            mp = lib.orc_col_mask(h, req, idx)
            mask = None
            if mp:
                nw = (ngroups + 31) // 32
                mask = np.ctypeslib.as_array((C.c_uint32 * nw).from_address(mp)).copy()
            if t == TypeId.STRUCT:
                # SUM_OVERFLOW: children {sum in the source type, overflow flag}, the mask on the struct
                ct = TypeId(lib.orc_col_child_type(h, req, idx))
                nb2 = lib.orc_col_bytes2(h, req, idx)
                flags = np.ctypeslib.as_array((C.c_uint8 * nb2).from_address(lib.orc_col_data2(h, req, idx))).copy() \
                    if nb2 else np.zeros(0, np.uint8)
                dec = ct in (TypeId.DECIMAL32, TypeId.DECIMAL64, TypeId.DECIMAL128)
                kids = [HostColumn(ct, int(ngroups), raw.view(STORAGE_DTYPE[ct]), None, 0, None, scale if dec else 0),
                        HostColumn(TypeId.BOOL8, int(ngroups), flags, None, 0, None, 0)]
                return HostColumn(t, int(ngroups), None, mask, 0, None, 0, kids)
            if t == TypeId.STRING:
                op = lib.orc_col_offsets(h, req, idx)
                offs = np.ctypeslib.as_array((C.c_int64 * (ngroups + 1)).from_address(op)).copy()
                return HostColumn(t, int(ngroups), raw, mask, 0, offs)
            # decimal columns (keys, SUM / MIN / MAX results) keep the scale of their source
            dec = t in (TypeId.DECIMAL32, TypeId.DECIMAL64, TypeId.DECIMAL128)
            return HostColumn(t, int(ngroups), raw.view(STORAGE_DTYPE[t]), mask, 0, None, scale if dec else 0)

        out_keys = [fetch(-1, i, getattr(keys[i], "scale", 0)) for i in range(len(keys))]
        out_res = [[fetch(q, a, getattr(vals, "scale", 0)) for a in range(len(aggs))]
                   for q, (vals, aggs) in enumerate(requests)]
        return out_keys, out_res
    finally:
        lib.orc_free(h)
