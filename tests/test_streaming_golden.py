"""The literal batches of the reference's streaming_groupby unit tests
(tests/golden/reference_streaming_cases.json, transcribed from
cpp/tests/groupby/streaming_groupby_test.cpp): the oracle over the concatenated batches must give
the outputs those tests state, and StreamingGroupBy over the batches (merge tests: two objects)
must equal both the stated output and the one-shot result, which is the rule
``verify_against_groupby`` applies in the reference."""
import json
import os

import numpy as np
import pytest

from cudf_b200.types import HostColumn, Kind, NullPolicy, TypeId, result_type
from oracle import oracle
from tests import helpers as H

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_streaming_cases.json")
with open(_PATH, encoding="utf-8") as _f:
    _CASES = json.load(_f)["cases"]


def _instances():
    for c in _CASES:
        for vt in (c["typed"] or [None]):
            types = list(c["value_types"]) if vt is None else [vt] + list(c["value_types"][1:])
            yield (c["name"] + (f"[{vt}]" if vt else ""), c, types)


INSTANCES = list(_instances())


def _batch_columns(case, vtypes, batch):
    nk = len(case["key_types"])
    cols = [H.make_column(batch[i], case["key_types"][i]) for i in range(nk)]
    cols += [H.make_column(batch[nk + j], vtypes[j]) for j in range(len(batch) - nk)]
    return cols


def _concat(case, vtypes):
    ncols = len(case["batches"][0])
    merged = [[x for b in case["batches"] for x in b[i]] for i in range(ncols)]
    return _batch_columns(case, vtypes, merged)


def _requests(case, cols):
    return [(cols[ci], [(Kind[agg], ddof)]) for ci, agg, ddof in case["requests"]]


def _expected_columns(case, vtypes):
    nk = len(case["key_types"])
    ek = [H.make_column(case["expect"]["keys"][i], case["key_types"][i]) for i in range(nk)]
    ev = []
    for (ci, agg, _), vals in zip(case["requests"], case["expect"]["vals"]):
        ev.append([H.make_column(vals, result_type(TypeId[vtypes[ci - nk]], Kind[agg]).name)])
    return ek, ev


@pytest.mark.parametrize("inst", [i for i in INSTANCES if i[1]["expect"] is not None], ids=lambda i: i[0])
def test_oracle_gives_the_outputs_the_reference_states(inst):
    _, case, vtypes = inst
    cols = _concat(case, vtypes)
    nk = len(case["key_types"])
    reqs = _requests(case, cols)
    got = oracle.groupby(cols[:nk], reqs, NullPolicy[case["null_policy"]])
    H.assert_same_result(got, _expected_columns(case, vtypes), reqs, check_nullable=False)


@pytest.mark.gpu
@pytest.mark.parametrize("inst", INSTANCES, ids=lambda i: i[0])
def test_streaming_groupby_matches_the_reference_cases(inst):
    import cudf_b200 as cb
    from cudf_b200.aggregation import Aggregation
    _, case, vtypes = inst
    nk = len(case["key_types"])
    policy = NullPolicy[case["null_policy"]]
    sreqs = [cb.StreamingAggregationRequest(ci, Aggregation(Kind[agg], ddof)) for ci, agg, ddof in case["requests"]]
    workers = case["workers"] or [0] * len(case["batches"])
    objs = [cb.StreamingGroupBy(list(range(nk)), sreqs, case["max_keys"], policy) for _ in range(max(workers) + 1)]
    for b, batch in enumerate(case["batches"]):
        objs[workers[b]].aggregate(cb.Table([cb.Column.from_host(c) for c in _batch_columns(case, vtypes, batch)]))
        if b in case["finalize_after"]:
            objs[workers[b]].finalize()  # must not consume or change the state
    for other in objs[1:]:
        objs[0].merge(other)
    res = objs[0].finalize()
    got = ([c.to_host() for c in res[0].columns()], [[c.to_host() for c in t.columns()] for t in res[1]])
    cols = _concat(case, vtypes)
    reqs = _requests(case, cols)
    H.assert_same_result(got, oracle.groupby(cols[:nk], reqs, policy), reqs)
    if case["expect"] is not None:
        H.assert_same_result(got, _expected_columns(case, vtypes), reqs, check_nullable=False)


@pytest.mark.gpu
def test_streaming_error_behaviour_follows_the_reference():
    """cpp/tests/groupby/streaming_groupby_test.cpp:647-666,834-853,876-882,1277-1291."""
    import cudf_b200 as cb
    from cudf_b200 import aggregation as agg

    def table(keys, vals):
        return cb.Table([cb.Column.from_host(HostColumn.from_numpy(np.array(keys, dtype=np.int32))),
                         cb.Column.from_host(HostColumn.from_numpy(np.array(vals, dtype=np.int32)))])
    sum_req = [cb.StreamingAggregationRequest(1, agg.sum())]
    with pytest.raises(ValueError):       # std::invalid_argument: an aggregation the streaming form does not serve
        cb.StreamingGroupBy([0], [cb.StreamingAggregationRequest(1, agg.median())], 1024)
    with pytest.raises(ValueError):       # a batch larger than max_distinct_keys
        cb.StreamingGroupBy([0], sum_req, 3).aggregate(table([1, 2, 3, 4, 5], [10, 20, 30, 40, 50]))
    s = cb.StreamingGroupBy([0], sum_req, 4)
    s.aggregate(table([0, 1, 2, 3], [10, 20, 30, 40]))
    with pytest.raises(cb.LogicError):    # one more distinct key than the capacity
        s.aggregate(table([4], [50]))
    with pytest.raises(cb.LogicError):    # finalize before any aggregate
        cb.StreamingGroupBy([0], sum_req, 1024).finalize()
