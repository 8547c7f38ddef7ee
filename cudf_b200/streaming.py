"""Batch-wise groupby with a persistent partial-aggregate state: the shape of
``cudf::groupby::streaming_groupby`` (cpp/include/cudf/groupby.hpp:478-598;
cpp/src/groupby/streaming_groupby/) over the state entry points of the C ABI
(b2_state_create / update / pack / merge / finalize).

Keys that pack into 64 bits keep one persistent hash table of partial aggregates on the device.
String, float and wider keys are kept as a TABLE of partial aggregates (one row per group: keys,
then Σx, n, Σx², min, max ... per source column); a new batch is aggregated on its own and the two
tables are merged by a reduction groupby over their concatenation (sum of sums, sum of counts, min
of mins ...), the way the reference's multi-partition path reduces partial aggregates
(python/cudf_polars/cudf_polars/streaming/actor_graph/groupby.py:339-456).  The compound results
(mean, M2, variance, std) are evaluated from the partial columns at ``finalize``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .aggregation import Aggregation
from .column import Column, Table
from .groupby import GroupBy, GroupByRequest, GroupByState, LogicError
from .types import Kind, NullPolicy, STORAGE_DTYPE, TypeId, is_duration, is_floating, result_type

_SUPPORTED = {Kind.SUM, Kind.SUM_OF_SQUARES, Kind.PRODUCT, Kind.MIN, Kind.MAX, Kind.COUNT_VALID, Kind.COUNT_ALL,
              Kind.MEAN, Kind.M2, Kind.VARIANCE, Kind.STD}

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


@dataclass
class StreamingAggregationRequest:
    """cudf::groupby::streaming_aggregation_request: which column of the batch table to aggregate, and how."""
    column_index: int
    aggregation: Aggregation


class StreamingGroupBy:
    """Feeds batches into a persistent partial-aggregate state; ``merge`` folds in another object's
    partial state; ``finalize`` produces the results without consuming the state."""

    def __init__(self, key_indices: Sequence[int], requests: Sequence[StreamingAggregationRequest],
                 max_distinct_keys: int, null_handling: NullPolicy = NullPolicy.EXCLUDE):
        if max_distinct_keys <= 0:
            raise ValueError("max_distinct_keys must be positive")
        for r in requests:
            if Kind(r.aggregation.kind) not in _SUPPORTED:
                raise ValueError(f"unsupported aggregation kind for streaming groupby: {Kind(r.aggregation.kind).name}")
        self._key_indices = list(key_indices)
        self._requests = list(requests)
        self._max = int(max_distinct_keys)
        self._policy = null_handling
        self._state: Optional[GroupByState] = None
        # row-keyed form (string / float / wide keys): a table of partial aggregates
        self._row_keyed: Optional[bool] = None
        self._pkeys: Optional[List[Column]] = None
        self._pcols: Dict[Tuple[int, Kind], Column] = {}
        self._src_type: Dict[int, TypeId] = {}
        self._src_scale: Dict[int, int] = {}
        self._src_nulls: Dict[int, bool] = {}
        # partial aggregates per source column: COUNT_VALID always (it decides validity), then what the requests need
        self._plan: List[Tuple[int, Kind]] = []
        for r in self._requests:
            for k in [Kind.COUNT_VALID] + _PARTIALS[Kind(r.aggregation.kind)]:
                if (r.column_index, k) not in self._plan:
                    self._plan.append((r.column_index, k))

    # ---------------------------------------------------------------------------------- packed keys
    def _bind(self, data: Table) -> Tuple[GroupBy, List[GroupByRequest]]:
        cols = data.columns()
        gb = GroupBy(Table([cols[i] for i in self._key_indices]), self._policy, expected_groups=self._max)
        reqs = [GroupByRequest(cols[r.column_index], [r.aggregation]) for r in self._requests]
        return gb, reqs

    def _keys_are_row_keyed(self, data: Table) -> bool:
        """The engine's rule: keys pack into 64 bits (one extra bit per nullable key under INCLUDE) unless
        one of them is a string or a float."""
        bits = 0
        for i in self._key_indices:
            c = data.columns()[i]
            if c.type_id == TypeId.STRING or is_floating(c.type_id):
                return True
            bits += 8 * np.dtype(STORAGE_DTYPE[c.type_id]).itemsize
            if self._policy == NullPolicy.INCLUDE and c.mask is not None:
                bits += 1
        return bits > 64

    # ---------------------------------------------------------------------------------- row keys
    def _aggregate_partials(self, keys: List[Column], sources: Dict[Tuple[int, Kind], Column], merging: bool):
        """One groupby producing the partial table: over a batch (``merging`` False: the plan's aggregations on
        the source columns) or over two concatenated partial tables (True: the reduction of each partial)."""
        reqs, order = [], []
        if not merging:
            by_col: Dict[int, List[Kind]] = {}
            for ci, k in self._plan:
                by_col.setdefault(ci, []).append(k)
            for ci, kinds in by_col.items():
                reqs.append(GroupByRequest(sources[(ci, Kind.COUNT_VALID)], [Aggregation(k) for k in kinds]))
                order += [(ci, k) for k in kinds]
        else:
            for key in self._plan:
                reqs.append(GroupByRequest(sources[key], [Aggregation(_MERGE[key[1]])]))
                order.append(key)
        okeys, ores = GroupBy(Table(keys), self._policy).aggregate(reqs)
        flat = [c for t in ores for c in t.columns()]
        out = {}
        for key, col in zip(order, flat):
            if key[1] in (Kind.COUNT_VALID, Kind.COUNT_ALL) and col.type_id != TypeId.INT64:
                col = _from_typed(_typed(col).to(torch.int64), TypeId.INT64, None)  # counts add up as INT64
            out[key] = col
        return okeys.columns(), out

    def _fold(self, keys: List[Column], pcols: Dict[Tuple[int, Kind], Column]):
        if self._pkeys is None or self._pkeys[0].size == 0:
            self._pkeys, self._pcols = keys, pcols
            return
        if keys[0].size == 0:
            return
        ck = [_concat(a, b) for a, b in zip(self._pkeys, keys)]
        cc = {key: _concat(self._pcols[key], pcols[key]) for key in self._plan}
        self._pkeys, self._pcols = self._aggregate_partials(ck, cc, merging=True)

    def _aggregate_rows(self, data: Table):
        cols = data.columns()
        for r in self._requests:
            c = cols[r.column_index]
            self._src_type[r.column_index] = c.type_id
            self._src_scale[r.column_index] = c.scale
            self._src_nulls[r.column_index] = self._src_nulls.get(r.column_index, False) or \
                (c.mask is not None and c.null_count != 0)
        keys = [cols[i] for i in self._key_indices]
        sources = {(ci, Kind.COUNT_VALID): cols[ci] for ci, _ in self._plan}
        bk, bp = self._aggregate_partials(keys, sources, merging=False)
        self._fold(bk, bp)

    def _finalize_rows(self):
        n = self._pkeys[0].size
        device = next((t.device for c in self._pkeys for t in (c.data, c.offsets) if t is not None), torch.device("cuda"))
        results = []
        for r in self._requests:
            ci, kind, ddof = r.column_index, Kind(r.aggregation.kind), r.aggregation.ddof
            st, has_nulls = self._src_type[ci], self._src_nulls[ci]
            rt = result_type(st, kind)
            cnt = _typed(self._pcols[(ci, Kind.COUNT_VALID)])
            some = (cnt > 0).to(torch.uint8)
            if kind in (Kind.COUNT_VALID, Kind.COUNT_ALL):
                src = cnt if kind == Kind.COUNT_VALID else _typed(self._pcols[(ci, Kind.COUNT_ALL)])
                col = _from_typed(src.to(torch.int32), TypeId.INT32, None)
            elif kind in (Kind.SUM, Kind.PRODUCT, Kind.MIN, Kind.MAX, Kind.SUM_OF_SQUARES):
                p = self._pcols[(ci, kind)]
                mask, nulls = None, 0
                if has_nulls:  # nullable iff the source has nulls (cpp/src/groupby/hash/output_utils.cu:61-68)
                    from .partition import bytes_to_mask
                    mask, nulls = bytes_to_mask(some)
                col = Column(p.type_id, p.size, p.data, mask, p.offset, nulls, None, TypeId.INT32, p.scale)
            elif kind == Kind.MEAN:
                s = _typed(self._pcols[(ci, Kind.SUM)])
                safe = torch.clamp(cnt, min=1)
                if is_duration(st):  # integer division in the source type
                    val = torch.div(s.to(torch.int64), safe, rounding_mode="trunc").to(s.dtype)
                else:
                    val = s.to(torch.float64) / safe.to(torch.float64)
                col = _from_typed(val, rt, some if has_nulls else None)
            else:  # M2, VARIANCE, STD (cpp/src/groupby/common/m2_var_std.cu:49-59,160-187)
                s = _typed(self._pcols[(ci, Kind.SUM)]).to(torch.float64)
                ss = _typed(self._pcols[(ci, Kind.SUM_OF_SQUARES)]).to(torch.float64)
                nf = torch.clamp(cnt, min=1).to(torch.float64)
                m2 = torch.where(cnt > 0, ss - s * s / nf, torch.zeros_like(ss))
                if kind == Kind.M2:
                    col = _from_typed(m2, TypeId.FLOAT64, None)
                else:
                    df = cnt - int(ddof)
                    ok = (cnt > 0) & (df > 0)
                    var = torch.where(ok, m2 / torch.clamp(df, min=1).to(torch.float64), torch.zeros_like(m2))
                    col = _from_typed(var if kind == Kind.VARIANCE else torch.sqrt(var), TypeId.FLOAT64, ok.to(torch.uint8))
            assert col.size == n
            results.append(Table([col]))
        return Table(list(self._pkeys)), results

    # ---------------------------------------------------------------------------------- public
    def aggregate(self, data: Table) -> None:
        """streaming_groupby::aggregate (groupby.hpp:539-541)."""
        if data.num_rows() > self._max:
            raise ValueError("a single batch may not exceed max_distinct_keys rows")
        if self._row_keyed is None:
            self._row_keyed = self._keys_are_row_keyed(data)
        if self._row_keyed:
            self._aggregate_rows(data)
        else:
            gb, reqs = self._bind(data)
            if self._state is None:
                self._state = GroupByState(gb, reqs)
            self._state.update(gb, reqs)
        self._check_capacity()

    def merge(self, other: "StreamingGroupBy") -> None:
        """streaming_groupby::merge (groupby.hpp:548-556): the other object is not modified."""
        if self._row_keyed is None:
            raise LogicError("merge() needs an object that has seen at least one aggregate() call")
        if other._row_keyed is None or other.distinct_keys() == 0:
            return
        if other.distinct_keys() > self._max:
            raise ValueError("the other object holds more distinct keys than max_distinct_keys")
        if self._row_keyed:
            for ci, flag in other._src_nulls.items():
                self._src_nulls[ci] = self._src_nulls.get(ci, False) or flag
            self._fold(list(other._pkeys), dict(other._pcols))
        else:
            records, counts = other._state.pack(1)
            self._state.merge(records, counts[0])
        self._check_capacity()

    def finalize(self):
        """streaming_groupby::finalize (groupby.hpp:566-568): (keys table, one results table per request)."""
        # before any aggregate() the reference throws; after batches that left no group (all keys
        # null under EXCLUDE, empty batches) it returns empty columns
        # (cpp/tests/groupby/streaming_groupby_test.cpp:514-538,876-882)
        if self._row_keyed is None:
            raise LogicError("no data has been accumulated")
        if self._row_keyed:
            return self._finalize_rows()
        return self._state.finalize()

    def distinct_keys(self) -> int:
        if self._row_keyed:
            return 0 if self._pkeys is None else self._pkeys[0].size
        return 0 if self._state is None else self._state.num_groups()

    def _check_capacity(self):
        if self.distinct_keys() > self._max:
            raise LogicError("cumulative distinct keys exceed max_distinct_keys")
