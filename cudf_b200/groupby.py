"""Host-side mirror of the reference's groupby API for the hash-aggregate path.

``GroupBy(keys, null_handling).aggregate(requests)`` has the shape and semantics of
``pylibcudf.groupby.GroupBy`` (python/pylibcudf/pylibcudf/groupby.pyx:134-214), which binds
``cudf::groupby::groupby`` (cpp/include/cudf/groupby.hpp:89-184).  Every call goes through the
C ABI of libb2groupby.so; there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from .aggregation import Aggregation
from .column import Column, Table, TorchAllocator, allocator_for
from .types import type_width, Kind, NullPolicy, TypeId


class LogicError(RuntimeError):
    """cudf::logic_error"""


class DataTypeError(TypeError):
    """cudf::data_type_error"""


class CudaError(RuntimeError):
    """cudf::cuda_error"""


class UnsupportedError(NotImplementedError):
    """The request is valid for the reference but is served by its sort-based path."""


_EXC = {
    _lib.Status.LOGIC_ERROR: LogicError, _lib.Status.INVALID_ARGUMENT: ValueError,
    _lib.Status.DATA_TYPE_ERROR: DataTypeError, _lib.Status.CUDA_ERROR: CudaError,
    _lib.Status.UNSUPPORTED: UnsupportedError, _lib.Status.OUT_OF_MEMORY: MemoryError,
    _lib.Status.INTERNAL_ERROR: RuntimeError,
}


def _check(status: int):
    if status != _lib.Status.SUCCESS:
        msg = _lib.load().b2_last_error().decode()
        raise _EXC.get(status, RuntimeError)(msg)


class GroupByRequest:
    """cudf::groupby::aggregation_request (cpp/include/cudf/groupby.hpp:54-57)."""

    def __init__(self, values: Column, aggregations: Sequence[Aggregation]):
        self._values = values
        self._aggregations = list(aggregations)


def _requests_to_c(requests: Sequence[GroupByRequest], keep: list):
    arr = (_lib.AggregationRequest * max(1, len(requests)))()
    for i, r in enumerate(requests):
        aggs = (_lib.Aggregation * max(1, len(r._aggregations)))()
        for j, a in enumerate(r._aggregations):
            aggs[j] = _lib.Aggregation(int(a.kind), int(a.ddof))
        keep.append(aggs)
        arr[i].values = r._values.c_view(keep)
        arr[i].num_aggregations = len(r._aggregations)
        arr[i].aggregations = aggs
    keep.append(arr)
    return arr


def _adopt_column(oc: _lib.OwnedColumn, alloc: TorchAllocator) -> Column:
    data = alloc.adopt(oc.data)
    mask = alloc.adopt(oc.null_mask)
    # a call that allocated its result before it knew the group count hands over buffers larger than the
    # column: the column's tensors are views of the part that belongs to it
    width = type_width(oc.type_id)
    if data is not None and width:
        used = (oc.size * width + 3) // 4 * 4
        if data.numel() > max(used, 8):
            data = data[:max(used, 8)]
    if mask is not None:
        used = max(1, (oc.size + 511) // 512) * 64
        if mask.numel() > used:
            mask = mask[:used]
    if oc.type_id in (int(TypeId.STRUCT), int(TypeId.DICTIONARY32)):  # children {sum, overflow} / {indices, keys}
        kids = [_adopt_column(oc.children[i], alloc) for i in range(oc.num_children)]
        oc.null_mask = None
        return Column(oc.type_id, oc.size, None, mask, 0, oc.null_count, children=kids)
    offsets, offs_t = None, TypeId.INT32
    if oc.num_children:
        child = oc.children[0]
        offsets = alloc.adopt(child.data)
        offs_t = TypeId(child.type_id)
        child.data = None
    oc.data = None
    oc.null_mask = None
    return Column(oc.type_id, oc.size, data, mask, 0, oc.null_count, offsets, offs_t, oc.scale)


def _adopt_result(res: _lib.GroupbyResult, alloc: TorchAllocator) -> Tuple[Table, List[Table]]:
    lib = _lib.load()
    try:
        keys = Table([_adopt_column(res.keys[k], alloc) for k in range(res.num_keys)])
        results = []
        for q in range(res.num_requests):
            results.append(Table([_adopt_column(res.results[q][a], alloc) for a in range(res.num_results[q])]))
        return keys, results
    finally:
        lib.b2_result_free(C.byref(res))


class CallStats:
    def __init__(self, s: _lib.CallStats):
        self.kernel_launches = s.kernel_launches
        self.table_attempts = s.table_attempts
        self.table_capacity = s.table_capacity
        self.scratch_bytes = s.scratch_bytes
        self.used_shared_table = bool(s.used_shared_table)
        self.aggregate_kernel_ms = float(s.aggregate_kernel_ms)

    def __repr__(self):
        return (f"CallStats(kernel_launches={self.kernel_launches}, table_attempts={self.table_attempts}, "
                f"table_capacity={self.table_capacity}, scratch_bytes={self.scratch_bytes}, "
                f"used_shared_table={self.used_shared_table}, aggregate_kernel_ms={self.aggregate_kernel_ms:.4f})")


def last_call_stats() -> CallStats:
    s = _lib.CallStats()
    _lib.load().b2_get_last_stats(C.byref(s))
    return CallStats(s)


class GroupBy:
    """Groups values by keys and computes aggregations on those groups.

    Parameters mirror ``pylibcudf.groupby.GroupBy.__init__`` (groupby.pyx:134-142): ``keys`` is the
    table of key columns, ``null_handling`` decides whether rows with a null key are dropped
    (EXCLUDE, default) or grouped (INCLUDE).  Extras of this engine: ``expected_groups`` (sizing
    hint), ``row_filters`` (validity masks a row must pass: a fused ``drop_nulls``),
    ``table_variant`` (0 auto, 1 global-memory table only, 3 shared-memory table with hashing only,
    4 / 5 the lean float-mean kernel with register tiles / with the bulk-copy tile ring, 6 / 7 always /
    never the radix-partitioned path for very many groups, 8 STRING keys through dictionary ids whatever the
    row count).
    """

    def __init__(self, keys: Table, null_handling: NullPolicy = NullPolicy.EXCLUDE, *,
                 expected_groups: int = 0, row_filters: Sequence[Column] = (), table_variant: int = 0,
                 shared_table_bytes: int = 0):
        lib = _lib.load()
        self._keys = keys
        self._keep: list = []
        n = keys.num_columns()
        views = (_lib.ColumnView * max(1, n))()
        for i, c in enumerate(keys.columns()):
            views[i] = c.c_view(self._keep)
        opts = _lib.GroupbyOptions()
        opts.expected_groups = int(expected_groups)
        opts.table_variant = int(table_variant)
        opts.shared_table_bytes = int(shared_table_bytes)
        filt = [c for c in row_filters if c.mask is not None]
        opts.num_row_filters = len(filt)
        if filt:
            masks = (C.c_void_p * len(filt))(*[c.mask.data_ptr() for c in filt])
            offs = (C.c_int32 * len(filt))(*[c.offset for c in filt])
            opts.row_filter_masks = masks
            opts.row_filter_offsets = offs
            self._keep += [masks, offs, filt]
        handle = C.c_void_p()
        _check(lib.b2_groupby_create(views, n, int(null_handling), C.byref(opts), C.byref(handle)))
        self._handle = handle
        self._device = keys.columns()[0].data.device if n and keys.columns()[0].data is not None else torch.device("cuda")

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h and _lib is not None and getattr(_lib, "_lib", None) is not None:  # not during interpreter shutdown
            _lib._lib.b2_groupby_destroy(h)
            self._handle = None

    def aggregate(self, requests: Sequence[GroupByRequest]) -> Tuple[Table, List[Table]]:
        """Returns (table of unique keys, one table of result columns per request), groups in
        arbitrary order (cpp/include/cudf/groupby.hpp:139-150)."""
        lib = _lib.load()
        keep: list = []
        creqs = _requests_to_c(requests, keep)
        alloc = allocator_for(self._device)
        res = _lib.GroupbyResult()
        stream = torch.cuda.current_stream(self._device).cuda_stream
        _check(lib.b2_groupby_aggregate(self._handle, creqs, len(requests), C.c_void_p(stream),
                                        C.byref(alloc.struct), C.byref(res)))
        return _adopt_result(res, alloc)


class GroupByState:
    """Partial-aggregate state: the local pass, the partition by owner, the merge and the
    finalisation of a multi-GPU (or batch-wise) groupby — see include/b2_groupby.h."""

    def __init__(self, gb: GroupBy, requests: Sequence[GroupByRequest]):
        lib = _lib.load()
        self._gb = gb
        self._keep: list = []
        creqs = _requests_to_c(requests, self._keep)
        handle = C.c_void_p()
        _check(lib.b2_state_create(gb._handle, creqs, len(requests), C.byref(handle)))
        self._handle = handle
        self._device = gb._device
        self._nreq = len(requests)

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h and _lib is not None and getattr(_lib, "_lib", None) is not None:  # not during interpreter shutdown
            _lib._lib.b2_state_destroy(h)
            self._handle = None

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self._device).cuda_stream)

    def update(self, gb: Optional[GroupBy] = None, requests: Optional[Sequence[GroupByRequest]] = None):
        """Aggregates the rows of ``gb``'s keys / ``requests``' values into the state."""
        lib = _lib.load()
        gb = gb or self._gb
        keep: list = []
        if requests is None:
            creqs = self._keep[-1]
        else:
            creqs = _requests_to_c(requests, keep)
        _check(lib.b2_state_update(self._handle, gb._handle, creqs, self._nreq, self._stream()))

    @property
    def record_bytes(self) -> int:
        return _lib.load().b2_state_record_bytes(self._handle)

    def pack(self, num_parts: int) -> Tuple[torch.Tensor, List[int]]:
        """Partial records grouped by owner partition: (uint8 tensor of records, records per part).
        The tensor is owned by the caller."""
        lib = _lib.load()
        ptr = C.c_void_p()
        nbytes = C.c_size_t()
        counts = (C.c_int64 * num_parts)()
        alloc = allocator_for(self._device)
        _check(lib.b2_state_pack(self._handle, num_parts, self._stream(), C.byref(alloc.struct), C.byref(ptr),
                                 C.byref(nbytes), counts))
        buf = alloc.adopt(ptr.value)
        return buf[:nbytes.value], [int(c) for c in counts]

    def chunk_bytes(self, chunk_records: int) -> int:
        return int(_lib.load().b2_state_chunk_bytes(self._handle, int(chunk_records)))

    def pack_chunks(self, num_parts: int, chunk_records: int) -> torch.Tensor:
        """Fixed-size partition of the partial records (one chunk per destination, no host sync)."""
        out = torch.empty(num_parts * self.chunk_bytes(chunk_records), dtype=torch.uint8, device=self._device)
        _check(_lib.load().b2_state_pack_chunks(self._handle, num_parts, int(chunk_records), self._stream(),
                                                C.c_void_p(out.data_ptr())))
        return out

    def merge_chunks(self, chunks: torch.Tensor, num_chunks: int, chunk_records: int):
        chunks = chunks.contiguous()
        self._chunks_keepalive = chunks
        _check(_lib.load().b2_state_merge_chunks(self._handle, C.c_void_p(chunks.data_ptr()), int(num_chunks),
                                                 int(chunk_records), self._stream()))

    def merge(self, records: torch.Tensor, num_records: int):
        lib = _lib.load()
        records = records.contiguous()
        _check(lib.b2_state_merge(self._handle, C.c_void_p(records.data_ptr()), int(num_records), self._stream()))

    def reset(self, expected_groups: int = 0):
        _check(_lib.load().b2_state_reset(self._handle, int(expected_groups), self._stream()))

    def num_groups(self) -> int:
        out = C.c_int64()
        _check(_lib.load().b2_state_num_groups(self._handle, self._stream(), C.byref(out)))
        return int(out.value)

    def finalize(self) -> Tuple[Table, List[Table]]:
        lib = _lib.load()
        alloc = allocator_for(self._device)
        res = _lib.GroupbyResult()
        _check(lib.b2_state_finalize(self._handle, self._stream(), C.byref(alloc.struct), C.byref(res)))
        return _adopt_result(res, alloc)
