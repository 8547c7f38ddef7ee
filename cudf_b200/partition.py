"""``hash_partition``: mirror of ``pylibcudf.partitioning.hash_partition`` /
``cudf::hash_partition`` (cpp/include/cudf/partitioning.hpp, cpp/src/partitioning/partitioning.cu:950-975)
for fixed-width tables, through the C ABI (b2_hash_partition)."""
from __future__ import annotations

import ctypes as C
from typing import List, Tuple

import torch

from . import _lib
from .column import Column, Table, TorchAllocator
from .groupby import _check


def hash_partition(table: Table, num_key_columns: int, num_partitions: int) -> Tuple[Table, List[int]]:
    """Reorders the rows so that partition p occupies rows [offsets[p], offsets[p+1]); the first
    ``num_key_columns`` columns are hashed.  Returns (partitioned table, offsets of num_partitions+1 entries)."""
    lib = _lib.load()
    cols = table.columns()
    keep: list = []
    views = (_lib.ColumnView * len(cols))()
    for i, c in enumerate(cols):
        views[i] = c.c_view(keep)
    device = cols[0].data.device if cols[0].data is not None else torch.device("cuda")
    alloc = TorchAllocator(device)
    out = (_lib.OwnedColumn * len(cols))()
    offsets = (C.c_int64 * (num_partitions + 1))()
    stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    _check(lib.b2_hash_partition(views, len(cols), num_key_columns, num_partitions, stream, C.byref(alloc.struct),
                                 out, offsets))
    res = []
    for i in range(len(cols)):
        oc = out[i]
        res.append(Column(oc.type_id, oc.size, alloc.adopt(oc.data), alloc.adopt(oc.null_mask), 0, oc.null_count))
    return Table(res), [int(o) for o in offsets]
