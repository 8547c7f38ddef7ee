"""Type ids, aggregation kinds and the host-side (numpy) Arrow-layout column.

The numeric values are those of the reference's enums so that a binding can pass them through
unchanged: ``cudf::type_id`` (cpp/include/cudf/types.hpp:185-217), ``cudf::aggregation::Kind``
(cpp/include/cudf/aggregation.hpp:78-121), ``cudf::null_policy`` (cpp/include/cudf/types.hpp:115-118).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np


class TypeId(enum.IntEnum):
    EMPTY = 0
    INT8 = 1
    INT16 = 2
    INT32 = 3
    INT64 = 4
    UINT8 = 5
    UINT16 = 6
    UINT32 = 7
    UINT64 = 8
    FLOAT32 = 9
    FLOAT64 = 10
    BOOL8 = 11
    TIMESTAMP_DAYS = 12
    TIMESTAMP_SECONDS = 13
    TIMESTAMP_MILLISECONDS = 14
    TIMESTAMP_MICROSECONDS = 15
    TIMESTAMP_NANOSECONDS = 16
    DURATION_DAYS = 17
    DURATION_SECONDS = 18
    DURATION_MILLISECONDS = 19
    DURATION_MICROSECONDS = 20
    DURATION_NANOSECONDS = 21
    DICTIONARY32 = 22
    STRING = 23
    LIST = 24
    DECIMAL32 = 25
    DECIMAL64 = 26
    DECIMAL128 = 27
    STRUCT = 28


class Kind(enum.IntEnum):
    SUM = 0
    SUM_OVERFLOW = 1   # struct {sum: the source type, overflow: BOOL8}
    PRODUCT = 2
    MIN = 3
    MAX = 4
    COUNT_VALID = 5
    COUNT_ALL = 6
    SUM_OF_SQUARES = 9
    MEAN = 10
    M2 = 11
    VARIANCE = 12
    STD = 13
    # kinds the reference serves on its sort path only; accepted by the API so that the
    # "unsupported" status can be reported the way an adapter needs it
    MEDIAN = 14
    ARGMAX = 16
    ARGMIN = 17
    NUNIQUE = 18
    NTH_ELEMENT = 19


class NullPolicy(enum.IntEnum):
    EXCLUDE = 0
    INCLUDE = 1


# storage dtype of each fixed-width type id
STORAGE_DTYPE = {
    TypeId.INT8: np.int8, TypeId.INT16: np.int16, TypeId.INT32: np.int32, TypeId.INT64: np.int64,
    TypeId.UINT8: np.uint8, TypeId.UINT16: np.uint16, TypeId.UINT32: np.uint32,
    TypeId.UINT64: np.uint64, TypeId.FLOAT32: np.float32, TypeId.FLOAT64: np.float64,
    TypeId.BOOL8: np.uint8,
    TypeId.TIMESTAMP_DAYS: np.int32, TypeId.TIMESTAMP_SECONDS: np.int64,
    TypeId.TIMESTAMP_MILLISECONDS: np.int64, TypeId.TIMESTAMP_MICROSECONDS: np.int64,
    TypeId.TIMESTAMP_NANOSECONDS: np.int64,
    TypeId.DURATION_DAYS: np.int32, TypeId.DURATION_SECONDS: np.int64,
    TypeId.DURATION_MILLISECONDS: np.int64, TypeId.DURATION_MICROSECONDS: np.int64,
    TypeId.DURATION_NANOSECONDS: np.int64,
    TypeId.DECIMAL32: np.int32, TypeId.DECIMAL64: np.int64,
    # a 16-byte two's-complement integer, little endian: the unsigned low word, then the signed high word
    TypeId.DECIMAL128: np.dtype([("lo", "<u8"), ("hi", "<i8")]),
}


def int128_array(values) -> np.ndarray:
    """Python integers -> an array of the DECIMAL128 storage type (values wrap modulo 2^128)."""
    out = np.zeros(len(values), dtype=STORAGE_DTYPE[TypeId.DECIMAL128])
    for i, v in enumerate(values):
        u = int(v) & ((1 << 128) - 1)
        out["lo"][i] = u & 0xFFFFFFFFFFFFFFFF
        hi = u >> 64
        out["hi"][i] = hi - (1 << 64) if hi >= (1 << 63) else hi
    return out


def int128_list(arr: np.ndarray) -> list:
    """The Python integers of an array of the DECIMAL128 storage type."""
    return [(int(h) << 64) + int(l) for l, h in zip(arr["lo"].tolist(), arr["hi"].tolist())]

_NUMPY_TO_TYPE = {
    np.dtype(np.int8): TypeId.INT8, np.dtype(np.int16): TypeId.INT16,
    np.dtype(np.int32): TypeId.INT32, np.dtype(np.int64): TypeId.INT64,
    np.dtype(np.uint8): TypeId.UINT8, np.dtype(np.uint16): TypeId.UINT16,
    np.dtype(np.uint32): TypeId.UINT32, np.dtype(np.uint64): TypeId.UINT64,
    np.dtype(np.float32): TypeId.FLOAT32, np.dtype(np.float64): TypeId.FLOAT64,
    np.dtype(np.bool_): TypeId.BOOL8,
}


def type_width(t: int) -> int:
    """Bytes per element of a fixed-width type id, 0 for the others."""
    t = TypeId(t)
    return np.dtype(STORAGE_DTYPE[t]).itemsize if t in STORAGE_DTYPE else 0


def is_floating(t: int) -> bool:
    return TypeId(t) in (TypeId.FLOAT32, TypeId.FLOAT64)


def is_duration(t: int) -> bool:
    return TypeId.DURATION_DAYS <= TypeId(t) <= TypeId.DURATION_NANOSECONDS


def is_timestamp(t: int) -> bool:
    return TypeId.TIMESTAMP_DAYS <= TypeId(t) <= TypeId.TIMESTAMP_NANOSECONDS


def is_decimal(t: int) -> bool:
    return TypeId(t) in (TypeId.DECIMAL32, TypeId.DECIMAL64, TypeId.DECIMAL128)


def result_type(source: int, kind: int) -> TypeId:
    """Result element type of aggregation ``kind`` over ``source``
    (cpp/include/cudf/detail/aggregation/aggregation.hpp:884-1013)."""
    source, kind = TypeId(source), Kind(kind)
    if kind in (Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.ARGMAX, Kind.ARGMIN):
        return TypeId.INT32
    if kind in (Kind.MIN, Kind.MAX):
        return source
    if kind == Kind.SUM_OVERFLOW:
        return TypeId.STRUCT  # children {sum: source, overflow: BOOL8} (aggregation.hpp:990-995)
    if kind == Kind.SUM:
        # decimals keep their type and scale (aggregation.hpp:956-963)
        return source if (is_floating(source) or is_duration(source) or is_decimal(source)) else TypeId.INT64
    if kind in (Kind.SUM_OF_SQUARES, Kind.PRODUCT):
        return source if is_floating(source) else TypeId.INT64
    if kind == Kind.MEAN:
        return source if is_duration(source) else TypeId.FLOAT64
    return TypeId.FLOAT64


def pack_mask(valid: np.ndarray, offset: int = 0) -> np.ndarray:
    """Boolean validity array -> cudf bitmask words (uint32, bit i%32 of word i//32, LSB first,
    1 = valid; cpp/include/cudf/utilities/bit.hpp:47-104).  ``offset`` leading bits are set valid.
    The word count is padded to a multiple of 16 words (64 bytes) like
    cudf::bitmask_allocation_size_bytes (cpp/include/cudf/null_mask.hpp:52-57)."""
    valid = np.asarray(valid, dtype=bool)
    if offset:
        valid = np.concatenate([np.ones(offset, dtype=bool), valid])
    nbits = valid.size
    nwords = max(16, ((nbits + 31) // 32 + 15) // 16 * 16)
    bits = np.zeros(nwords * 32, dtype=np.uint8)
    bits[:nbits] = valid
    return np.packbits(bits, bitorder="little").view(np.uint32).copy()


def unpack_mask(mask: Optional[np.ndarray], size: int, offset: int = 0) -> np.ndarray:
    """Bitmask words -> boolean validity array of ``size`` elements (all True for ``None``)."""
    if mask is None:
        return np.ones(size, dtype=bool)
    bits = np.unpackbits(np.ascontiguousarray(mask).view(np.uint8), bitorder="little")
    return bits[offset:offset + size].astype(bool)


@dataclass
class HostColumn:
    """A column in the reference's Arrow layout held in numpy arrays on the host
    (fields of cudf::column_view, cpp/include/cudf/column/column_view.hpp:236-243,469)."""

    type_id: TypeId
    size: int
    data: Optional[np.ndarray]            # fixed width: elements (incl. the ``offset`` prefix); STRING: chars (uint8)
    mask: Optional[np.ndarray] = None     # uint32 words or None
    offset: int = 0
    offsets: Optional[np.ndarray] = None  # STRING: int32 or int64, offset+size+1 entries
    scale: int = 0                        # DECIMAL32/64: value = data * 10**scale (cpp/include/cudf/types.hpp data_type)
    children: Optional[list] = None       # STRUCT: the child columns (``data`` is None)

    @property
    def null_count(self) -> int:
        return int(self.size - unpack_mask(self.mask, self.size, self.offset).sum())

    @staticmethod
    def from_numpy(values, valid=None, type_id: Optional[int] = None, offset: int = 0, scale: int = 0) -> "HostColumn":
        """Fixed-width column from an array; ``valid`` is an optional boolean array (False = null).
        ``offset`` > 0 builds a sliced view: the first ``offset`` elements are padding."""
        values = np.ascontiguousarray(values)
        if type_id is None:
            type_id = _NUMPY_TO_TYPE[values.dtype]
        type_id = TypeId(type_id)
        store = np.dtype(STORAGE_DTYPE[type_id])
        if values.dtype == np.bool_:
            values = values.astype(np.uint8)
        if values.dtype != store:
            values = values.astype(store)
        n = values.size
        if offset:
            values = np.concatenate([np.full(offset, 77, dtype=store), values])
        mask = None
        if valid is not None:
            mask = pack_mask(np.asarray(valid, dtype=bool), offset)
        return HostColumn(type_id, n, values, mask, offset, None, int(scale))

    @staticmethod
    def from_dictionary(values, valid=None, index_type: int = TypeId.INT32, offset: int = 0) -> "HostColumn":
        """DICTIONARY32 column of fixed-width values: children {indices, sorted unique keys}
        (cpp/include/cudf/dictionary/dictionary_column_view.hpp:29-57).  The index of a null row is arbitrary."""
        values = np.ascontiguousarray(values)
        ok = np.ones(values.size, dtype=bool) if valid is None else np.asarray(valid, dtype=bool)
        keys = np.unique(values[ok])
        idx = np.searchsorted(keys, values) if keys.size else np.zeros(values.size, dtype=np.int64)
        idx = np.where(ok, np.minimum(idx, max(keys.size - 1, 0)), 0)
        indices = HostColumn.from_numpy(idx.astype(STORAGE_DTYPE[TypeId(index_type)]), type_id=index_type, offset=offset)
        indices.offset = 0  # the parent's offset applies to the indices (their prefix is padding)
        indices.size = values.size + offset
        parent = HostColumn(TypeId.DICTIONARY32, values.size, None,
                            None if valid is None else pack_mask(ok, offset), offset, None, 0,
                            [indices, HostColumn.from_numpy(keys)])
        return parent

    @staticmethod
    def from_strings(strings: Sequence[Optional[str]], large_offsets: bool = False) -> "HostColumn":
        """STRING column from Python strings (None = null), UTF-8 bytes, INT32 or INT64 offsets
        (cpp/include/cudf/strings/strings_column_view.hpp:53)."""
        enc = [b"" if s is None else (s if isinstance(s, bytes) else s.encode("utf-8")) for s in strings]
        lens = np.fromiter((len(b) for b in enc), dtype=np.int64, count=len(enc))
        offs = np.zeros(len(enc) + 1, dtype=np.int64)
        np.cumsum(lens, out=offs[1:])
        chars = np.frombuffer(b"".join(enc), dtype=np.uint8).copy() if len(enc) else np.zeros(0, np.uint8)
        valid = np.array([s is not None for s in strings], dtype=bool)
        mask = None if valid.all() else pack_mask(valid)
        return HostColumn(TypeId.STRING, len(enc), chars, mask, 0,
                          offs if large_offsets else offs.astype(np.int32))

    # -- readers used by tests ------------------------------------------------------------
    def valid(self) -> np.ndarray:
        return unpack_mask(self.mask, self.size, self.offset)

    def values(self) -> np.ndarray:
        """Elements of a fixed-width column (without the slice prefix)."""
        return self.data[self.offset:self.offset + self.size]

    def to_pylist(self) -> list:
        v = self.valid()
        if self.type_id == TypeId.STRING:
            o = self.offsets[self.offset:self.offset + self.size + 1].astype(np.int64)
            raw = self.data.tobytes()
            return [raw[o[i]:o[i + 1]] if v[i] else None for i in range(self.size)]
        vals = self.values()
        return [vals[i].item() if v[i] else None for i in range(self.size)]
