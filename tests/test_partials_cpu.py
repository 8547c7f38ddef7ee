"""Host-side logic of the partial-aggregate table (no GPU): which keys are row-keyed, and which partial
aggregates a set of requests needs."""
import numpy as np
import torch

from cudf_b200.column import Column
from cudf_b200.partials import PartialTable, keys_are_row_keyed
from cudf_b200.types import Kind, NullPolicy, TypeId


def _col(type_id, n=4, nullable=False, width=None):
    width = width or {TypeId.INT8: 1, TypeId.INT16: 2, TypeId.INT32: 4, TypeId.INT64: 8, TypeId.FLOAT32: 4,
                      TypeId.FLOAT64: 8, TypeId.DECIMAL64: 8}.get(type_id, 1)
    mask = torch.full((64,), 255, dtype=torch.uint8) if nullable else None
    offsets = torch.zeros((n + 1) * 4, dtype=torch.uint8) if type_id == TypeId.STRING else None
    return Column(type_id, n, torch.zeros(n * width, dtype=torch.uint8), mask, 0, 0, offsets)


def test_keys_pack_into_64_bits_like_the_engine():
    assert not keys_are_row_keyed([_col(TypeId.INT32), _col(TypeId.INT32)], NullPolicy.EXCLUDE)
    assert not keys_are_row_keyed([_col(TypeId.INT64)], NullPolicy.INCLUDE)
    assert not keys_are_row_keyed([_col(TypeId.DECIMAL64)], NullPolicy.EXCLUDE)
    # a nullable 64-bit key needs a 65th bit under INCLUDE only
    assert keys_are_row_keyed([_col(TypeId.INT64, nullable=True)], NullPolicy.INCLUDE)
    assert not keys_are_row_keyed([_col(TypeId.INT64, nullable=True)], NullPolicy.EXCLUDE)
    assert keys_are_row_keyed([_col(TypeId.INT64), _col(TypeId.INT8)], NullPolicy.EXCLUDE)
    # strings and floats compare by value (NaN == NaN, +0 == -0) or by bytes: never packed
    assert keys_are_row_keyed([_col(TypeId.STRING)], NullPolicy.EXCLUDE)
    assert keys_are_row_keyed([_col(TypeId.FLOAT32)], NullPolicy.EXCLUDE)


def test_partial_plan_follows_the_decomposition_of_the_reference():
    """MEAN -> SUM + COUNT_VALID; M2 / VARIANCE / STD -> SUM_OF_SQUARES + SUM + COUNT_VALID
    (cpp/src/groupby/hash/extract_single_pass_aggs.cpp:63-109); one partial column per (source, kind)."""
    pt = PartialTable([("a", Kind.MEAN, 1), ("a", Kind.SUM, 1), ("a", Kind.STD, 1), ("b", Kind.MAX, 1),
                       ("b", Kind.COUNT_ALL, 1)], NullPolicy.EXCLUDE)
    assert pt.plan == [("a", Kind.COUNT_VALID), ("a", Kind.SUM), ("a", Kind.SUM_OF_SQUARES),
                       ("b", Kind.COUNT_VALID), ("b", Kind.MAX), ("b", Kind.COUNT_ALL)]
    assert pt.size == 0


def test_partial_table_rejects_kinds_without_a_partial_form():
    import pytest
    from cudf_b200.groupby import UnsupportedError
    with pytest.raises(UnsupportedError):
        PartialTable([("a", Kind.MEDIAN, 1)], NullPolicy.EXCLUDE)
