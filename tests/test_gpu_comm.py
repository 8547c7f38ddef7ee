"""b2_groupby_aggregate_multi through the C ABI on ONE GPU: a one-rank NCCL communicator sends every
partial record to itself, which runs the whole native plan (local aggregate, partition by owner,
ncclSend / ncclRecv, merge, finalise) on a single-GPU box.  Both exchange forms: fixed-size chunks
(few groups) and exact sizes after a chunk overflow (more groups than a chunk holds)."""
import ctypes as C

import numpy as np
import pytest

import workloads
from cudf_b200.types import HostColumn, Kind, NullPolicy
from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _multi(comm, keys, requests, policy=NullPolicy.EXCLUDE, row_filters=()):
    import torch
    import cudf_b200 as cb
    from cudf_b200 import _lib
    from cudf_b200.aggregation import Aggregation
    from cudf_b200.column import allocator_for
    from cudf_b200.groupby import GroupBy, _adopt_result, _check, _requests_to_c
    lib = _lib.load()
    dkeys = cb.Table([cb.Column.from_host(k) for k in keys])
    cache, reqs = {}, []
    for vals, aggs in requests:
        cache.setdefault(id(vals), cb.Column.from_host(vals))
        reqs.append(cb.GroupByRequest(cache[id(vals)], [Aggregation(Kind(a[0]), a[1]) if isinstance(a, tuple)
                                                         else Aggregation(Kind(a)) for a in aggs]))
    gb = GroupBy(dkeys, policy, row_filters=[cache[id(f)] for f in row_filters])
    keep = []
    creqs = _requests_to_c(reqs, keep)
    alloc = allocator_for(gb._device)
    res = _lib.GroupbyResult()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _check(lib.b2_groupby_aggregate_multi(comm, gb._handle, creqs, len(reqs), stream, C.byref(alloc.struct), C.byref(res)))
    okeys, ores = _adopt_result(res, alloc)
    return [c.to_host() for c in okeys.columns()], [[c.to_host() for c in t.columns()] for t in ores]


@pytest.fixture(scope="module")
def comm():
    from cudf_b200 import _lib
    from cudf_b200.groupby import _check
    lib = _lib.load()
    ident = (C.c_uint8 * 128)()
    _check(lib.b2_comm_unique_id(ident))
    handle = C.c_void_p()
    _check(lib.b2_comm_create(ident, 0, 1, C.byref(handle)))
    yield handle
    lib.b2_comm_destroy(handle)


def _check_against_oracle(comm, w):
    got = _multi(comm, w.keys, w.requests, w.null_policy, w.row_filters)
    fm = [f.mask for f in w.row_filters if f.mask is not None]
    exp = oracle.groupby(w.keys, w.requests, w.null_policy, row_filters=fm)
    H.assert_same_result(got, exp, w.requests, scales=H.result_scales(w.keys, w.requests, w.null_policy, fm))
    return got


def test_one_rank_native_plan_small_states_travel_as_chunks(comm):
    got = _check_against_oracle(comm, workloads.make(2, 300_000))
    assert got[0][0].size == 10_000
    _check_against_oracle(comm, workloads.make(1, 200_000))


def test_one_rank_native_plan_falls_back_to_exact_sizes(comm):
    # ~59K groups: more than the 16384 records a chunk holds
    w = workloads.make(3, 300_000, scale_domain=True)
    got = _check_against_oracle(comm, w)
    assert got[0][0].size > 16384
    _check_against_oracle(comm, workloads.make(4, 300_000, scale_domain=True))
    _check_against_oracle(comm, workloads.make(2, 100_000))   # small again: back to chunks


def test_row_keyed_requests_are_refused_before_any_communication(comm):
    import cudf_b200 as cb
    w = workloads.make(5, 5_000, scale_domain=True)
    with pytest.raises(cb.UnsupportedError):
        _multi(comm, w.keys, w.requests, w.null_policy)
