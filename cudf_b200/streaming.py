"""Batch-wise groupby with a persistent partial-aggregate state: the shape of
``cudf::groupby::streaming_groupby`` (cpp/include/cudf/groupby.hpp:478-598;
cpp/src/groupby/streaming_groupby/) over the state entry points of the C ABI
(b2_state_create / update / pack / merge / finalize).

Keys that pack into 64 bits keep one persistent hash table of partial aggregates on the device.
String, float and wider keys are kept as a table of partial aggregates that a reduction groupby
folds batch by batch (cudf_b200/partials.py)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

from .aggregation import Aggregation
from .column import Table
from .groupby import GroupBy, GroupByRequest, GroupByState, LogicError
from .partials import PartialTable, keys_are_row_keyed
from .types import Kind, NullPolicy

_SUPPORTED = {Kind.SUM, Kind.SUM_OF_SQUARES, Kind.PRODUCT, Kind.MIN, Kind.MAX, Kind.COUNT_VALID, Kind.COUNT_ALL,
              Kind.MEAN, Kind.M2, Kind.VARIANCE, Kind.STD}


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
        self._row_keyed: Optional[bool] = None       # decided by the first batch's key types
        self._state: Optional[GroupByState] = None   # packed keys: the persistent device table
        self._partials = PartialTable([(r.column_index, r.aggregation.kind, r.aggregation.ddof) for r in requests],
                                      null_handling)  # string / float / wide keys

    def _bind(self, data: Table) -> Tuple[GroupBy, List[GroupByRequest]]:
        cols = data.columns()
        gb = GroupBy(Table([cols[i] for i in self._key_indices]), self._policy, expected_groups=self._max)
        reqs = [GroupByRequest(cols[r.column_index], [r.aggregation]) for r in self._requests]
        return gb, reqs

    def aggregate(self, data: Table) -> None:
        """streaming_groupby::aggregate (groupby.hpp:539-541)."""
        if data.num_rows() > self._max:
            raise ValueError("a single batch may not exceed max_distinct_keys rows")
        cols = data.columns()
        keys = [cols[i] for i in self._key_indices]
        if self._row_keyed is None:
            self._row_keyed = keys_are_row_keyed(keys, self._policy)
        if self._row_keyed:
            self._partials.add_batch(keys, {r.column_index: cols[r.column_index] for r in self._requests})
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
            self._partials.absorb(other._partials)
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
            keys, results = self._partials.finalize()
            return Table(keys), [Table([c]) for c in results]
        return self._state.finalize()

    def distinct_keys(self) -> int:
        if self._row_keyed:
            return self._partials.size
        return 0 if self._state is None else self._state.num_groups()

    def _check_capacity(self):
        if self.distinct_keys() > self._max:
            raise LogicError("cumulative distinct keys exceed max_distinct_keys")
