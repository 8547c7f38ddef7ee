"""Pins the CPU oracle to the known-answer vectors of the reference's own groupby unit tests."""
import numpy as np
import pytest

from cudf_b200.types import HostColumn, Kind, NullPolicy, TypeId
from oracle import oracle
from tests import helpers as H

CASES = [inst for case in H.load_golden() for inst in H.golden_instances(case)]


@pytest.mark.parametrize("inst", CASES, ids=[c[0] for c in CASES])
def test_oracle_matches_reference_known_answers(inst):
    _, keys, vals, kind, ddof, policy, ekeys, evals = inst
    okeys, ores = oracle.groupby([keys], [(vals, [(kind, ddof)])], policy)
    og, oe = H.sort_order(okeys), H.sort_order([ekeys])
    H.assert_keys_equal(okeys, [ekeys], og, oe)
    # the reference's tests compare values with a 4-ULP tolerance
    # (cpp/include/cudf_test/column_utilities.hpp:37)
    H.assert_column_equal(ores[0][0], evals, og, oe, 1e-15 if evals.type_id == TypeId.FLOAT64 else 1e-6, "values")


def test_oracle_size_mismatch_message():
    k = HostColumn.from_numpy(np.arange(4, dtype=np.int32))
    v = HostColumn.from_numpy(np.arange(5, dtype=np.int32))
    with pytest.raises(oracle.OracleError, match="Size mismatch between request values and groupby keys."):
        oracle.groupby([k], [(v, [Kind.SUM])])


def test_oracle_invalid_combination():
    k = HostColumn.from_numpy(np.arange(3, dtype=np.int32))
    v = HostColumn.from_strings(["a", "b", "c"])
    with pytest.raises(oracle.OracleError, match="Invalid type/aggregation combination."):
        oracle.groupby([k], [(v, [Kind.SUM])])


def test_oracle_sliced_m2_matches_unsliced():
    # cpp/tests/groupby/m2_tests.cpp:218 SlicedColumnsInput: rows 10..24 of a longer column
    keys = [4, 3, 1, 2, 3, 1, 2, 2, 1, None, 3, 2, 4, 4]
    vals = [None, None, 0.0, 1.0, 2.0, 3.0, 4.0, "nan", 6.0, 7.0, 8.0, 9.0, 10.0, "nan"]
    k0, v0 = H.make_column(keys, "INT32"), H.make_column(vals, "FLOAT64")
    k1, v1 = H.make_column(keys, "INT32", offset=10), H.make_column(vals, "FLOAT64", offset=10)
    a = oracle.groupby([k0], [(v0, [Kind.M2])])
    b = oracle.groupby([k1], [(v1, [Kind.M2])])
    oa, ob = H.sort_order(a[0]), H.sort_order(b[0])
    H.assert_keys_equal(a[0], b[0], oa, ob)
    H.assert_column_equal(a[1][0][0], b[1][0][0], oa, ob, 0.0, "m2")
    got = H.take(a[1][0][0], oa)
    assert got[0] == 18.0 and np.isnan(got[1]) and got[2] == 18.0 and np.isnan(got[3])


def test_oracle_threads_agree():
    rng = np.random.default_rng(5)
    n = 300_000
    k = HostColumn.from_numpy(rng.integers(0, 1000, n).astype(np.int64))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.05)
    a = oracle.groupby([k], [(v, [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN, Kind.MIN, Kind.MAX])])
    b = oracle.groupby([k], [(v, [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN, Kind.MIN, Kind.MAX])], threads=4)
    oa, ob = H.sort_order(a[0]), H.sort_order(b[0])
    H.assert_keys_equal(a[0], b[0], oa, ob)
    for x, y in zip(a[1][0], b[1][0]):
        H.assert_column_equal(x, y, oa, ob, 1e-15, "threads")


def test_oracle_decimal_sum_keeps_type_and_wraps_like_the_representation():
    """Fixed point SUM accumulates in the column's own representation type
    (cpp/include/cudf/detail/aggregation/aggregation.hpp:956-963): a DECIMAL32 sum wraps at 32 bits,
    and the scale of keys and results is the source's."""
    k = HostColumn.from_numpy(np.array([7, 7, 7, 9], dtype=np.int64), type_id=TypeId.DECIMAL64, scale=-3)
    v = HostColumn.from_numpy(np.array([2**31 - 1, 5, 10, -4], dtype=np.int32), type_id=TypeId.DECIMAL32, scale=2)
    okeys, ores = oracle.groupby([k], [(v, [Kind.SUM, Kind.MIN, Kind.MAX, Kind.COUNT_VALID])])
    assert okeys[0].type_id == TypeId.DECIMAL64 and okeys[0].scale == -3
    got = {int(key): [c.values()[i].item() for c in ores[0]] for i, key in enumerate(okeys[0].values())}
    wrapped = int(np.array([2**31 - 1 + 15], dtype=np.int64).astype(np.int32)[0])
    assert got == {7: [wrapped, 5, 2**31 - 1, 3], 9: [-4, -4, -4, 1]}
    assert [c.type_id for c in ores[0]] == [TypeId.DECIMAL32, TypeId.DECIMAL32, TypeId.DECIMAL32, TypeId.INT32]
    assert [c.scale for c in ores[0]] == [2, 2, 2, 0]
    with pytest.raises(oracle.OracleError, match="Invalid type/aggregation combination."):
        oracle.groupby([k], [(v, [Kind.PRODUCT])])
