"""StreamingGroupBy against the rules of the reference's streaming tests
(cpp/tests/groupby/streaming_groupby_test.cpp: MergeTwoObjects :300, NullKeysExcluded/Included :456,482,
MergeMeanTwoBatches :884, MergeCountTwoBatches :912, MergeVarianceTwoBatches :942, MultiColumnKeys :1248):
batches and merged partial states must equal a one-shot groupby of all rows."""
import numpy as np
import pytest

from cudf_b200.types import HostColumn, Kind, NullPolicy
from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu
KINDS = [Kind.SUM, Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.MEAN, Kind.MIN, Kind.MAX, Kind.VARIANCE, Kind.STD, Kind.M2,
         Kind.SUM_OF_SQUARES]


def _inputs(seed, n, nkeys=1):
    rng = np.random.default_rng(seed)
    # int32 + int16 keys: with one null bit each they still pack into 64 bits (a packed state takes many batches)
    keys = [HostColumn.from_numpy(rng.integers(0, 40, n).astype(np.int32 if i == 0 else np.int16),
                                  valid=rng.random(n) > 0.05) for i in range(nkeys)]
    v = HostColumn.from_numpy(rng.standard_normal(n) * 10, valid=rng.random(n) > 0.15)
    w = HostColumn.from_numpy(rng.integers(-50, 50, n).astype(np.int64))
    return keys, [v, w]


def _table(cols, lo, hi):
    import cudf_b200 as cb

    def cut(c):
        return HostColumn.from_numpy(c.values()[lo:hi], c.valid()[lo:hi] if c.mask is not None else None, type_id=c.type_id)
    return cb.Table([cb.Column.from_host(cut(c)) for c in cols])


def _host(res):
    return [c.to_host() for c in res[0].columns()], [[c.to_host() for c in t.columns()] for t in res[1]]


@pytest.mark.parametrize("policy", [NullPolicy.EXCLUDE, NullPolicy.INCLUDE])
@pytest.mark.parametrize("nkeys", [1, 2])
def test_batches_and_merge_equal_one_shot(policy, nkeys):
    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation
    n = 90_000
    keys, vals = _inputs(7 + nkeys, n, nkeys)
    cols = keys + vals
    sreqs = [cb.StreamingAggregationRequest(nkeys + i, Aggregation(k)) for i in range(2) for k in KINDS]
    a = cb.StreamingGroupBy(list(range(nkeys)), sreqs, 100_000, policy)
    b = cb.StreamingGroupBy(list(range(nkeys)), sreqs, 100_000, policy)
    a.aggregate(_table(cols, 0, 20_000))
    a.aggregate(_table(cols, 20_000, 50_000))
    b.aggregate(_table(cols, 50_000, 90_000))
    assert a.distinct_keys() > 0 and b.distinct_keys() > 0
    before = b.distinct_keys()
    a.merge(b)
    assert b.distinct_keys() == before          # the other object is not modified
    got = _host(a.finalize())
    reqs = [(vals[i], [k]) for i in range(2) for k in KINDS]
    exp = oracle.groupby(keys, reqs, policy)
    H.assert_same_result(got, exp, reqs, scales=H.result_scales(keys, reqs, policy))
    # finalize does not consume the state
    got2 = _host(a.finalize())
    H.assert_same_result(got2, exp, reqs, scales=H.result_scales(keys, reqs, policy))


def test_streaming_errors():
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg
    keys, vals = _inputs(3, 1000)
    sreq = [cb.StreamingAggregationRequest(1, agg.sum())]
    with pytest.raises(ValueError):
        cb.StreamingGroupBy([0], sreq, 0)
    with pytest.raises(ValueError):
        cb.StreamingGroupBy([0], [cb.StreamingAggregationRequest(1, agg.median())], 10)
    s = cb.StreamingGroupBy([0], sreq, 100)
    with pytest.raises(cb.LogicError):
        s.finalize()
    with pytest.raises(ValueError, match="single batch"):
        s.aggregate(_table(keys + vals, 0, 1000))
    t = cb.StreamingGroupBy([0], sreq, 10)       # 40 distinct keys do not fit 10
    with pytest.raises(cb.LogicError, match="max_distinct_keys"):
        for lo in range(0, 1000, 10):
            t.aggregate(_table(keys + vals, lo, lo + 10))


@pytest.mark.parametrize("policy", [NullPolicy.EXCLUDE, NullPolicy.INCLUDE])
def test_string_and_float_keys_take_many_batches_and_merge(policy):
    """Keys that do not pack into 64 bits are kept as a table of partial aggregates which is reduced batch by
    batch (cpp/tests/groupby/streaming_groupby_test.cpp:1043-1222 for string keys): the result must equal the
    one-shot groupby of all rows, for every aggregation kind, with null keys, null values, NaN keys."""
    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation
    rng = np.random.default_rng(19)
    n = 30_000
    pool = [f"key-{i:03d}-{'x' * (i % 7)}" for i in range(50)] + ["", "ü", "🙂"]
    sk = [pool[i] if rng.random() > 0.03 else None for i in rng.integers(0, len(pool), n)]
    fk = rng.integers(0, 4, n).astype(np.float32)
    fk[rng.random(n) < 0.05] = np.nan
    v = HostColumn.from_numpy(rng.standard_normal(n) * 10, valid=rng.random(n) > 0.15)
    w = HostColumn.from_numpy(rng.integers(-50, 50, n).astype(np.int64))
    d = HostColumn.from_numpy(rng.integers(0, 10**6, n).astype(np.int64), valid=rng.random(n) > 0.5,
                              type_id=cb.TypeId.DURATION_SECONDS)

    def cut(lo, hi):
        def fixed(c):
            return HostColumn.from_numpy(c.values()[lo:hi], c.valid()[lo:hi] if c.mask is not None else None,
                                         type_id=c.type_id)
        cols = [HostColumn.from_strings(sk[lo:hi]), HostColumn.from_numpy(fk[lo:hi]), fixed(v), fixed(w), fixed(d)]
        return cb.Table([cb.Column.from_host(c) for c in cols])

    sreqs = [cb.StreamingAggregationRequest(2 + i, Aggregation(k)) for i in range(2) for k in KINDS]
    sreqs += [cb.StreamingAggregationRequest(4, Aggregation(k)) for k in (Kind.SUM, Kind.MIN, Kind.MAX, Kind.MEAN,
                                                                           Kind.COUNT_VALID)]
    a = cb.StreamingGroupBy([0, 1], sreqs, 100_000, policy)
    b = cb.StreamingGroupBy([0, 1], sreqs, 100_000, policy)
    a.aggregate(cut(0, 7_000))
    a.aggregate(cut(7_000, 7_000))          # an empty batch
    a.aggregate(cut(7_000, 18_000))
    b.aggregate(cut(18_000, 30_000))
    before = b.distinct_keys()
    a.merge(b)
    assert b.distinct_keys() == before
    got = _host(a.finalize())
    keys = [HostColumn.from_strings(sk), HostColumn.from_numpy(fk)]
    reqs = [((v, w)[i], [k]) for i in range(2) for k in KINDS]
    reqs += [(d, [k]) for k in (Kind.SUM, Kind.MIN, Kind.MAX, Kind.MEAN, Kind.COUNT_VALID)]
    exp = oracle.groupby(keys, reqs, policy)
    H.assert_same_result(got, exp, reqs, scales=H.result_scales(keys, reqs, policy))
    assert a.distinct_keys() == exp[0][0].size
