"""A table of partial aggregates (one row per group: the keys, then n, Σx, Σx², min, max ... per source
column) and its reduction: the form in which groups whose keys do not pack into 64 bits (strings,
floats, wide composites) are carried between batches (streaming) and between ranks (multi-GPU).

Two partial tables meet by concatenation followed by a reduction groupby — sum of sums, sum of
counts, min of mins, max of maxes — the way the reference's multi-partition groupby reduces its
partial aggregates (python/cudf_polars/cudf_polars/streaming/actor_graph/groupby.py:339-456;
cpp/src/groupby/streaming_groupby/merge.cu:30-61).  The compound results (mean, M2, variance,
std) are evaluated from the partial columns at ``finalize``
(cpp/src/groupby/hash/hash_compound_agg_finalizer.cu:93-186, cpp/src/groupby/common/m2_var_std.cu:49-59,160-187).
Every aggregation runs through the CUDA engine (``GroupBy.aggregate``); torch only concatenates
buffers and evaluates the elementwise finalisers."""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .aggregation import Aggregation
from .column import Column, Table
from .groupby import GroupBy, GroupByRequest
from .types import Kind, NullPolicy, STORAGE_DTYPE, TypeId, is_duration, is_floating, result_type

# requested kind -> partial aggregates of the source column it is finalised from
# (cpp/src/groupby/hash/extract_single_pass_aggs.cpp:63-109)
_PARTIALS = {
    Kind.SUM: [Kind.SUM], Kind.PRODUCT: [Kind.PRODUCT], Kind.MIN: [Kind.MIN], Kind.MAX: [Kind.MAX],
    Kind.COUNT_VALID: [], Kind.COUNT_ALL: [Kind.COUNT_ALL], Kind.SUM_OF_SQUARES: [Kind.SUM_OF_SQUARES],
    Kind.MEAN: [Kind.SUM], Kind.M2: [Kind.SUM_OF_SQUARES, Kind.SUM],
    Kind.VARIANCE: [Kind.SUM_OF_SQUARES, Kind.SUM], Kind.STD: [Kind.SUM_OF_SQUARES, Kind.SUM],
}
# how a partial column is reduced when two partial tables meet
# (cpp/src/groupby/streaming_groupby/merge.cu:30-61)
_MERGE = {Kind.SUM: Kind.SUM, Kind.PRODUCT: Kind.PRODUCT, Kind.MIN: Kind.MIN, Kind.MAX: Kind.MAX,
          Kind.COUNT_VALID: Kind.SUM, Kind.COUNT_ALL: Kind.SUM, Kind.SUM_OF_SQUARES: Kind.SUM}

_TORCH = {np.dtype(np.int8): torch.int8, np.dtype(np.int16): torch.int16, np.dtype(np.int32): torch.int32,
          np.dtype(np.int64): torch.int64, np.dtype(np.uint8): torch.uint8, np.dtype(np.float32): torch.float32,
          np.dtype(np.float64): torch.float64}


def _typed(col: Column) -> torch.Tensor:
    """The elements of a fixed-width result column as a typed tensor (a view of its bytes)."""
    dt = _TORCH[np.dtype(STORAGE_DTYPE[col.type_id])]
    width = np.dtype(STORAGE_DTYPE[col.type_id]).itemsize
    if col.size == 0:
        return torch.zeros(0, dtype=dt, device=col.data.device if col.data is not None else "cuda")
    return col.data[col.offset * width:(col.offset + col.size) * width].view(dt)


def _valid_bytes(col: Column, device) -> torch.Tensor:
    from .partition import mask_to_bytes
    if col.mask is None or col.size == 0:
        return torch.ones(col.size, dtype=torch.uint8, device=device)
    return mask_to_bytes(col)


def _from_typed(values: torch.Tensor, type_id: TypeId, valid: Optional[torch.Tensor], scale: int = 0) -> Column:
    """A column from a typed tensor and optional validity bytes (1 = valid)."""
    from .partition import bytes_to_mask
    values = values.contiguous()
    mask, nulls = None, 0
    if valid is not None:
        mask, nulls = bytes_to_mask(valid.to(torch.uint8))
    raw = values.view(torch.uint8).reshape(-1) if values.numel() else torch.zeros(0, dtype=torch.uint8, device=values.device)
    return Column(type_id, values.numel(), raw, mask, 0, nulls, None, TypeId.INT32, scale)


def _finish(kind, ddof: int, result_type_id: TypeId, sums: Optional[Column], counts: Column,
            sum_sq: Optional[Column], nullable: bool) -> Column:
    """One finished result column from partial columns: the library's finishers (b2_finish_partial) — mean, M2,
    variance, standard deviation, counts as INT32, or (``kind`` None) only the validity a result takes from n."""
    import ctypes as C
    from . import _lib
    from .column import allocator_for
    from .groupby import _check
    lib = _lib.load()
    keep: list = []
    device = counts.data.device if counts.data is not None else torch.device("cuda")
    alloc = allocator_for(device)
    views = [(_lib.ColumnView * 1)(c.c_view(keep)) if c is not None else None for c in (sums, counts, sum_sq)]
    out = _lib.OwnedColumn()
    stream = torch.cuda.current_stream(device).cuda_stream
    _check(lib.b2_finish_partial(-1 if kind is None else int(kind), int(ddof), int(result_type_id), views[0], views[1],
                                 views[2], 1 if nullable else 0, C.c_void_p(stream), C.byref(alloc.struct), C.byref(out)))
    data = alloc.adopt(out.data)
    mask = alloc.adopt(out.null_mask)
    col = Column(out.type_id, out.size, data, mask, 0, out.null_count, None, TypeId.INT32, 0)
    out.data = None
    out.null_mask = None
    return col


def _concat(a: Column, b: Column) -> Column:
    """Rows of ``a`` followed by rows of ``b`` (same type)."""
    from .partition import bytes_to_mask
    device = next(t.device for t in (a.data, b.data, a.offsets, b.offsets, a.mask, b.mask) if t is not None)
    mask, nulls = None, 0
    if a.mask is not None or b.mask is not None:
        mask, nulls = bytes_to_mask(torch.cat([_valid_bytes(a, device), _valid_bytes(b, device)]))
    n = a.size + b.size
    if a.type_id == TypeId.STRING:
        def parts(c):
            od = torch.int64 if c.offsets_type == TypeId.INT64 else torch.int32
            offs = c.offsets.view(od)[c.offset:c.offset + c.size + 1].to(torch.int64)
            lo, hi = (int(offs[0]), int(offs[-1])) if c.size else (0, 0)
            chars = c.data[lo:hi] if c.data is not None else torch.zeros(0, dtype=torch.uint8, device=device)
            return chars, offs - lo
        ca, oa = parts(a)
        cb_, ob = parts(b)
        offs = torch.cat([oa, ob[1:] + oa[-1]]).contiguous()
        chars = torch.cat([ca, cb_]).contiguous()
        return Column(TypeId.STRING, n, chars, mask, 0, nulls, offs.view(torch.uint8), TypeId.INT64)
    width = np.dtype(STORAGE_DTYPE[a.type_id]).itemsize

    def body(c):
        if c.size == 0 or c.data is None:
            return torch.zeros(0, dtype=torch.uint8, device=device)
        return c.data[c.offset * width:(c.offset + c.size) * width]
    return Column(a.type_id, n, torch.cat([body(a), body(b)]).contiguous(), mask, 0, nulls, None, TypeId.INT32, a.scale)



def keys_are_row_keyed(keys: Sequence[Column], policy: NullPolicy) -> bool:
    """The engine's rule: keys pack into 64 bits (one extra bit per nullable key under INCLUDE) unless one
    of them is a string or a float.  Row-keyed tables cannot ship their slots as records."""
    bits = 0
    for c in keys:
        if c.type_id == TypeId.STRING or is_floating(c.type_id):
            return True
        bits += 8 * np.dtype(STORAGE_DTYPE[c.type_id]).itemsize
        if policy == NullPolicy.INCLUDE and c.mask is not None:
            bits += 1
    return bits > 64


class PartialTable:
    """``specs``: one (source id, kind, ddof) per requested aggregation, in output order; the source id is
    any hashable that names a value column (a column index, ``id(column)``)."""

    def __init__(self, specs: Sequence[Tuple[Hashable, Kind, int]], policy: NullPolicy, batch_options=None):
        from .groupby import UnsupportedError
        self.specs = [(s, Kind(k), int(d)) for s, k, d in specs]
        for _, k, _ in self.specs:
            if k not in _PARTIALS:
                raise UnsupportedError(f"aggregation {k.name} has no partial form")
        self.policy = policy
        self.batch_options = dict(batch_options or {})  # GroupBy options of the batch pass (row filters ...)
        self.keys: Optional[List[Column]] = None
        self.cols: Dict[Tuple[Hashable, Kind], Column] = {}
        self.src_type: Dict[Hashable, TypeId] = {}
        self.src_nulls: Dict[Hashable, bool] = {}
        # partial aggregates per source: COUNT_VALID always (it decides validity), then what the requests need
        self.plan: List[Tuple[Hashable, Kind]] = []
        for sid, kind, _ in self.specs:
            for k in [Kind.COUNT_VALID] + _PARTIALS[kind]:
                if (sid, k) not in self.plan:
                    self.plan.append((sid, k))

    @property
    def size(self) -> int:
        return 0 if self.keys is None else self.keys[0].size

    def _aggregate(self, keys: List[Column], sources: Dict, merging: bool):
        """One engine call producing a partial table: over a batch (``merging`` False: the plan's aggregations of
        the source columns, ``sources`` keyed by source id) or over concatenated partial rows (True: the
        reduction of each partial column, ``sources`` keyed like ``plan``)."""
        reqs, order = [], []
        if not merging:
            by_src: Dict[Hashable, List[Kind]] = {}
            for sid, k in self.plan:
                by_src.setdefault(sid, []).append(k)
            for sid, kinds in by_src.items():
                reqs.append(GroupByRequest(sources[sid], [Aggregation(k) for k in kinds]))
                order += [(sid, k) for k in kinds]
        else:
            for key in self.plan:
                reqs.append(GroupByRequest(sources[key], [Aggregation(_MERGE[key[1]])]))
                order.append(key)
        okeys, ores = GroupBy(Table(keys), self.policy, **({} if merging else self.batch_options)).aggregate(reqs)
        flat = [c for t in ores for c in t.columns()]
        out = {}
        for key, col in zip(order, flat):
            if key[1] in (Kind.COUNT_VALID, Kind.COUNT_ALL) and col.type_id != TypeId.INT64:
                col = _from_typed(_typed(col).to(torch.int64), TypeId.INT64, None)  # counts add up as INT64
            out[key] = col
        return okeys.columns(), out

    def note_sources(self, sources: Dict[Hashable, Column]) -> None:
        for sid, c in sources.items():
            self.src_type[sid] = c.type_id
            self.src_nulls[sid] = self.src_nulls.get(sid, False) or (c.mask is not None and c.null_count != 0)

    def add_batch(self, keys: List[Column], sources: Dict[Hashable, Column]) -> None:
        """Aggregates one batch of rows and folds it into the table."""
        self.note_sources(sources)
        bk, bp = self._aggregate(keys, sources, merging=False)
        self.fold(bk, bp)

    def fold(self, keys: List[Column], pcols: Dict[Tuple[Hashable, Kind], Column]) -> None:
        """Adds partial rows (keys may repeat keys already held)."""
        if self.keys is None or self.keys[0].size == 0:
            self.keys, self.cols = list(keys), dict(pcols)
            return
        if keys[0].size == 0:
            return
        ck = [_concat(a, b) for a, b in zip(self.keys, keys)]
        cc = {key: _concat(self.cols[key], pcols[key]) for key in self.plan}
        self.keys, self.cols = self._aggregate(ck, cc, merging=True)

    def absorb(self, other: "PartialTable") -> None:
        for sid, flag in other.src_nulls.items():
            self.src_nulls[sid] = self.src_nulls.get(sid, False) or flag
        for sid, t in other.src_type.items():
            self.src_type.setdefault(sid, t)
        if other.keys is not None:
            self.fold(list(other.keys), dict(other.cols))

    def columns(self) -> List[Column]:
        """The partial columns in ``plan`` order."""
        return [self.cols[key] for key in self.plan]

    def reduce_rows(self, keys: List[Column], cols: Sequence[Column]) -> None:
        """Replaces the table by the reduction of partial rows whose keys may repeat (rows received from
        several ranks), ``cols`` in ``plan`` order."""
        if keys[0].size == 0:
            self.keys, self.cols = list(keys), dict(zip(self.plan, cols))
            return
        self.keys, self.cols = self._aggregate(list(keys), dict(zip(self.plan, cols)), merging=True)

    def finalize(self, detect_nulls: bool = False) -> Tuple[List[Column], List[Column]]:
        """(key columns, one result column per spec).  ``detect_nulls``: also treat a source as having nulls
        when a group holds no valid value of it (partial rows that came from other ranks)."""
        n = self.size
        results = []
        for sid, kind, ddof in self.specs:
            st = self.src_type[sid]
            rt = result_type(st, kind)
            cnt = _typed(self.cols[(sid, Kind.COUNT_VALID)])
            has_nulls = self.src_nulls.get(sid, False)
            if detect_nulls and not has_nulls and n:
                has_nulls = bool((cnt == 0).any())
            count_col = self.cols[(sid, Kind.COUNT_VALID)]
            if kind in (Kind.COUNT_VALID, Kind.COUNT_ALL):
                src = count_col if kind == Kind.COUNT_VALID else self.cols[(sid, Kind.COUNT_ALL)]
                col = _finish(Kind.COUNT_VALID, 0, TypeId.INT32, None, src, None, False)
            elif kind in (Kind.SUM, Kind.PRODUCT, Kind.MIN, Kind.MAX, Kind.SUM_OF_SQUARES):
                p = self.cols[(sid, kind)]
                mask, nulls = None, 0
                if has_nulls:  # nullable iff the source has nulls (cpp/src/groupby/hash/output_utils.cu:61-68)
                    carrier = _finish(None, 0, TypeId.INT8, None, count_col, None, True)
                    mask, nulls = carrier.mask, carrier.null_count
                col = Column(p.type_id, p.size, p.data, mask, p.offset, nulls, None, TypeId.INT32, p.scale)
            elif kind == Kind.MEAN:
                col = _finish(Kind.MEAN, 0, rt, self.cols[(sid, Kind.SUM)], count_col, None, has_nulls)
            else:  # M2, VARIANCE, STD
                col = _finish(kind, int(ddof), TypeId.FLOAT64, self.cols[(sid, Kind.SUM)], count_col,
                              self.cols[(sid, Kind.SUM_OF_SQUARES)], True)
            assert col.size == n
            results.append(col)
        return list(self.keys), results
