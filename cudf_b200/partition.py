"""``hash_partition``: mirror of ``pylibcudf.partitioning.hash_partition`` /
``cudf::hash_partition`` (cpp/include/cudf/partitioning.hpp:97-108, cpp/src/partitioning/partitioning.cu:876-975)
for tables of fixed-width and STRING columns, through the C ABI (b2_hash_partition), plus the
validity bitmask <-> byte helpers a row exchange needs."""
from __future__ import annotations

import ctypes as C
from typing import List, Tuple

import torch

from . import _lib
from .column import Column, Table, allocator_for
from .groupby import _check
from .types import TypeId

HASH_IDENTITY, HASH_MURMUR3 = 0, 1   # cudf::hash_id (cpp/include/cudf/partitioning.hpp:32-35)
DEFAULT_HASH_SEED = 0                # cpp/include/cudf/hashing.hpp:29


def hash_partition(table: Table, columns_to_hash, num_partitions: int, hash_function: int = HASH_MURMUR3,
                   seed: int = DEFAULT_HASH_SEED) -> Tuple[Table, List[int]]:
    """Reorders the rows so that partition p occupies rows [offsets[p], offsets[p+1]).
    ``columns_to_hash`` is the list of column indices whose values decide the partition, like the
    reference's argument (cpp/include/cudf/partitioning.hpp), or an int k meaning the first k columns;
    ``hash_function`` / ``seed`` as in the reference (MurmurHash3_x86_32 with seed 0 by default), and
    the partition of every row is the reference's.
    Returns (partitioned table with the input's column order, offsets of num_partitions+1 entries).
    No columns to hash, no partitions, no rows or no columns give an empty table of the same column
    types (cpp/tests/partitioning/hash_partition_test.cpp:72-142); a column index outside the table
    raises IndexError (std::out_of_range there, :48-58)."""
    lib = _lib.load()
    cols = table.columns()
    if isinstance(columns_to_hash, int):
        hashed = list(range(columns_to_hash))
    else:
        hashed = [int(i) for i in columns_to_hash]
    if any(i < 0 or i >= len(cols) for i in hashed):
        raise IndexError("columns_to_hash names a column the table does not have")
    order = hashed + [i for i in range(len(cols)) if i not in hashed]  # the C entry point hashes the leading columns
    keep: list = []
    views = (_lib.ColumnView * max(1, len(cols)))()
    for j, i in enumerate(order):
        views[j] = cols[i].c_view(keep)
    device = next((c.data.device for c in cols if c.data is not None), torch.device("cuda"))
    alloc = allocator_for(device)
    out = (_lib.OwnedColumn * max(1, len(cols)))()
    offsets = (C.c_int64 * (num_partitions + 1))()
    stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    _check(lib.b2_hash_partition(views, len(cols), len(hashed), num_partitions, int(hash_function), int(seed) & 0xFFFFFFFF,
                                 stream, C.byref(alloc.struct), out, offsets))
    res: List[Column] = [None] * len(cols)  # type: ignore[list-item]
    for j, i in enumerate(order):
        oc = out[j]
        offs, offs_t = None, TypeId.INT32
        if oc.num_children:
            child = oc.children[0]
            offs = alloc.adopt(child.data)
            offs_t = TypeId(child.type_id)
            child.data = None
        res[i] = Column(oc.type_id, oc.size, alloc.adopt(oc.data), alloc.adopt(oc.null_mask), 0, oc.null_count,
                        offs, offs_t, oc.scale)
        oc.data = None
        oc.null_mask = None
        lib.b2_column_free(C.byref(oc), C.byref(alloc.struct), stream)  # host arrays of the descriptor
    return Table(res), [int(o) for o in offsets]


def mask_to_bytes(col: Column) -> torch.Tensor:
    """One byte per row (1 = valid) from the column's validity bitmask."""
    out = torch.empty(max(col.size, 1), dtype=torch.uint8, device=col.mask.device)
    stream = C.c_void_p(torch.cuda.current_stream(out.device).cuda_stream)
    _check(_lib.load().b2_mask_to_bytes(C.c_void_p(col.mask.data_ptr()), col.offset, col.size, stream,
                                        C.c_void_p(out.data_ptr())))
    return out[:col.size]


def bytes_to_mask(valid: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """cudf bitmask words (as a uint8 tensor, 64-byte padded) and the null count from validity bytes."""
    n = valid.numel()
    valid = valid.contiguous()
    words = max(16, ((n + 31) // 32 + 15) // 16 * 16)
    mask = torch.zeros(words * 4, dtype=torch.uint8, device=valid.device)
    nulls = torch.zeros(1, dtype=torch.int32, device=valid.device)
    stream = C.c_void_p(torch.cuda.current_stream(valid.device).cuda_stream)
    _check(_lib.load().b2_bytes_to_mask(C.c_void_p(valid.data_ptr() if n else mask.data_ptr()), n, stream,
                                        C.c_void_p(mask.data_ptr()), C.c_void_p(nulls.data_ptr())))
    return mask, int(nulls.item())
