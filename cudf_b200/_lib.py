"""ctypes binding of libb2groupby.so: the structs and prototypes of include/b2_groupby.h.

There is no fallback: if the CUDA library is missing, importing a compute entry point raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb2groupby.so")


class Status:
    SUCCESS, LOGIC_ERROR, INVALID_ARGUMENT, DATA_TYPE_ERROR, CUDA_ERROR, UNSUPPORTED, OUT_OF_MEMORY, INTERNAL_ERROR = range(8)


class ColumnView(C.Structure):
    pass


ColumnView._fields_ = [
    ("type_id", C.c_int32), ("scale", C.c_int32), ("size", C.c_int32), ("null_count", C.c_int32),
    ("data", C.c_void_p), ("null_mask", C.c_void_p), ("offset", C.c_int32), ("num_children", C.c_int32),
    ("children", C.POINTER(ColumnView)),
]


class Aggregation(C.Structure):
    _fields_ = [("kind", C.c_int32), ("ddof", C.c_int32)]


class AggregationRequest(C.Structure):
    _fields_ = [("values", ColumnView), ("num_aggregations", C.c_int32), ("aggregations", C.POINTER(Aggregation))]


ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p)
FREE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p)


class Allocator(C.Structure):
    _fields_ = [("allocate", ALLOC_FN), ("deallocate", FREE_FN), ("ctx", C.c_void_p)]


class OwnedColumn(C.Structure):
    pass


OwnedColumn._fields_ = [
    ("type_id", C.c_int32), ("scale", C.c_int32), ("size", C.c_int32), ("null_count", C.c_int32),
    ("data", C.c_void_p), ("data_bytes", C.c_size_t), ("null_mask", C.c_void_p), ("null_mask_bytes", C.c_size_t),
    ("num_children", C.c_int32), ("children", C.POINTER(OwnedColumn)),
]


class GroupbyResult(C.Structure):
    _fields_ = [
        ("num_groups", C.c_int32), ("num_keys", C.c_int32), ("keys", C.POINTER(OwnedColumn)),
        ("num_requests", C.c_int32), ("num_results", C.POINTER(C.c_int32)),
        ("results", C.POINTER(C.POINTER(OwnedColumn))), ("allocator", Allocator), ("stream", C.c_void_p),
    ]


class GroupbyOptions(C.Structure):
    _fields_ = [
        ("expected_groups", C.c_int64), ("table_variant", C.c_int32), ("shared_table_bytes", C.c_int32),
        ("num_row_filters", C.c_int32), ("row_filter_masks", C.POINTER(C.c_void_p)),
        ("row_filter_offsets", C.POINTER(C.c_int32)),
    ]


class CallStats(C.Structure):
    _fields_ = [("kernel_launches", C.c_int32), ("table_attempts", C.c_int32), ("table_capacity", C.c_int64),
                ("scratch_bytes", C.c_int64), ("used_shared_table", C.c_int32), ("aggregate_kernel_ms", C.c_float)]


# every symbol include/b2_groupby.h declares: name -> (restype, argtypes)
PROTOTYPES = {
    "b2_groupby_create": (C.c_int, [C.POINTER(ColumnView), C.c_int32, C.c_int32, C.POINTER(GroupbyOptions),
                                    C.POINTER(C.c_void_p)]),
    "b2_groupby_aggregate": (C.c_int, [C.c_void_p, C.POINTER(AggregationRequest), C.c_int32, C.c_void_p,
                                       C.POINTER(Allocator), C.POINTER(GroupbyResult)]),
    "b2_groupby_destroy": (None, [C.c_void_p]),
    "b2_result_free": (None, [C.POINTER(GroupbyResult)]),
    "b2_state_create": (C.c_int, [C.c_void_p, C.POINTER(AggregationRequest), C.c_int32, C.POINTER(C.c_void_p)]),
    "b2_state_update": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(AggregationRequest), C.c_int32, C.c_void_p]),
    "b2_state_record_bytes": (C.c_int32, [C.c_void_p]),
    "b2_state_pack": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.POINTER(Allocator), C.POINTER(C.c_void_p),
                            C.POINTER(C.c_size_t), C.POINTER(C.c_int64)]),
    "b2_state_chunk_bytes": (C.c_int64, [C.c_void_p, C.c_int64]),
    "b2_state_pack_chunks": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p]),
    "b2_state_merge_chunks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_void_p]),
    "b2_state_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "b2_state_reset": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p]),
    "b2_state_num_groups": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]),
    "b2_state_finalize": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(Allocator), C.POINTER(GroupbyResult)]),
    "b2_state_destroy": (None, [C.c_void_p]),
    "b2_hash_partition": (C.c_int, [C.POINTER(ColumnView), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_uint32,
                                    C.c_void_p, C.POINTER(Allocator), C.POINTER(OwnedColumn), C.POINTER(C.c_int64)]),
    "b2_mask_to_bytes": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b2_bytes_to_mask": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2_finish_partial": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(ColumnView), C.POINTER(ColumnView),
                                    C.POINTER(ColumnView), C.c_int32, C.c_void_p, C.POINTER(Allocator),
                                    C.POINTER(OwnedColumn)]),
    "b2_column_free": (None, [C.POINTER(OwnedColumn), C.POINTER(Allocator), C.c_void_p]),
    "b2_groupby_aggregate_noalloc": (C.c_int, [C.c_void_p, C.POINTER(AggregationRequest), C.c_int32, C.c_void_p,
                                               C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                               C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int32),
                                               C.POINTER(C.c_int32)]),
    "b2_comm_unique_id": (C.c_int, [C.c_void_p]),
    "b2_comm_create": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "b2_comm_adopt": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "b2_comm_destroy": (None, [C.c_void_p]),
    "b2_groupby_aggregate_multi": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(AggregationRequest), C.c_int32, C.c_void_p,
                                             C.POINTER(Allocator), C.POINTER(GroupbyResult)]),
    "b2_last_error": (C.c_char_p, []),
    "b2_version": (C.c_char_p, []),
    "b2_get_last_stats": (None, [C.POINTER(CallStats)]),
}

_lib = None


class LibraryMissing(ImportError):
    pass


def load() -> C.CDLL:
    """Loads the CUDA library; raises LibraryMissing (never falls back) when it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} is not built; run `python -m cudf_b200.build` (needs nvcc). "
                "There is no CPU fallback for the groupby path.")
        lib = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError here = the .so does not export a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib
