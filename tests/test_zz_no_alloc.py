"""The aggregate entry point that allocates no device memory, checked against the regular one.

Some callers cannot allocate while they run: a serving loop that must never hit the implicit
device synchronisation of cudaMalloc, a plug-in living inside a framework that owns all device
memory and only lends fixed buffers, a process whose pool is frozen.  For them
``b2_groupby_aggregate_noalloc`` works entirely inside caller-provided output buffers plus one
fixed scratch array inside the library (8 MiB per GPU, see include/b2_groupby.h).

This file is collected last on purpose: if it fails, a run that stops at the first failure has
already run every other test.  It passes alone in a fresh process as well as after the others.
"""
import ctypes as C

import numpy as np
import pytest

from cudf_b200.types import HostColumn, Kind, NullPolicy, STORAGE_DTYPE, TypeId, result_type
from tests import helpers as H

pytestmark = pytest.mark.gpu


def device_memory_in_use():
    """(bytes in use, bytes reserved) of the device's default stream-ordered pool — where every
    temporary of this library comes from — and the driver's count of free device bytes.  torch's own
    counters would not do: they only see torch's caching allocator, which the library never uses."""
    from cuda.bindings import runtime as rt
    err, dev = rt.cudaGetDevice()
    assert err == rt.cudaError_t.cudaSuccess
    err, pool = rt.cudaDeviceGetDefaultMemPool(dev)
    assert err == rt.cudaError_t.cudaSuccess
    vals = []
    for attr in (rt.cudaMemPoolAttr.cudaMemPoolAttrUsedMemCurrent, rt.cudaMemPoolAttr.cudaMemPoolAttrReservedMemCurrent):
        err, v = rt.cudaMemPoolGetAttribute(pool, attr)
        assert err == rt.cudaError_t.cudaSuccess
        vals.append(int(v))
    err, free, _total = rt.cudaMemGetInfo()
    assert err == rt.cudaError_t.cudaSuccess
    return vals[0], vals[1], int(free)


def run_noalloc(keys, requests, policy, max_groups, warmed_up=False):
    """Calls b2_groupby_aggregate_noalloc through the C ABI; output buffers are plain torch tensors
    allocated by the test (the caller's job), returned as host columns.  Checks that the call left
    the device's memory accounting untouched: the default pool always, the driver's free-byte count
    once a first call has loaded the kernels (``warmed_up``)."""
    import torch
    import cudf_b200 as cb
    from cudf_b200 import _lib
    from cudf_b200.aggregation import Aggregation
    from cudf_b200.groupby import GroupBy, _check, _requests_to_c

    lib = _lib.load()
    dkeys = cb.Table([cb.Column.from_host(k) for k in keys])
    dvals = {}
    reqs = []
    for vals, aggs in requests:
        if id(vals) not in dvals:
            dvals[id(vals)] = cb.Column.from_host(vals)
        reqs.append(cb.GroupByRequest(dvals[id(vals)], [Aggregation(Kind(a[0]), a[1]) if isinstance(a, tuple)
                                                         else Aggregation(Kind(a)) for a in aggs]))
    gb = GroupBy(dkeys, policy)
    keep = []
    creqs = _requests_to_c(reqs, keep)
    words = (max_groups + 31) // 32

    def buf(type_id):
        width = np.dtype(STORAGE_DTYPE[TypeId(type_id)]).itemsize if TypeId(type_id) in STORAGE_DTYPE else 8
        return torch.empty(max_groups * width + 8, dtype=torch.uint8, device="cuda")

    key_bufs = [buf(k.type_id) for k in keys]
    key_masks = [torch.empty(words * 4, dtype=torch.uint8, device="cuda") for _ in keys]
    rtypes = [result_type(v.type_id, (a[0] if isinstance(a, tuple) else a)) for v, aggs in requests for a in aggs]
    res_bufs = [buf(t) for t in rtypes]
    res_masks = [torch.empty(words * 4, dtype=torch.uint8, device="cuda") for _ in rtypes]
    nk, nr = len(keys), len(rtypes)
    c_key_data = (C.c_void_p * nk)(*[t.data_ptr() for t in key_bufs])
    c_key_masks = (C.c_void_p * nk)(*[t.data_ptr() for t in key_masks])
    c_res_data = (C.c_void_p * nr)(*[t.data_ptr() for t in res_bufs])
    c_res_masks = (C.c_void_p * nr)(*[t.data_ptr() for t in res_masks])
    ngroups = C.c_int32()
    nulls = (C.c_int32 * (nk + nr))()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    used0, reserved0, free0 = device_memory_in_use()
    _check(lib.b2_groupby_aggregate_noalloc(gb._handle, creqs, len(reqs), stream, max_groups, c_key_data, c_key_masks,
                                            c_res_data, c_res_masks, C.byref(ngroups), nulls))
    used1, reserved1, free1 = device_memory_in_use()
    assert torch.cuda.memory_allocated() == before
    assert (used1, reserved1) == (used0, reserved0), "the call touched the default memory pool"
    if warmed_up:
        assert free1 == free0, "device memory was allocated or released during the call"
    G = ngroups.value

    def column(t, data, mask, null_count, nullable):
        dt = np.dtype(STORAGE_DTYPE[TypeId(t)])
        vals = data.cpu().numpy()[: G * dt.itemsize].view(dt).copy()
        m = mask.cpu().numpy().view(np.uint32)[: max(1, (G + 31) // 32)].copy() if nullable else None
        col = HostColumn(TypeId(t), G, vals, m, 0)
        assert col.null_count == null_count
        return col

    out_keys = [column(k.type_id, key_bufs[i], key_masks[i], nulls[i],
                       policy == NullPolicy.INCLUDE and k.mask is not None) for i, k in enumerate(keys)]
    out_res, i = [], 0
    for vals, aggs in requests:
        row = []
        for a in aggs:
            kind = a[0] if isinstance(a, tuple) else a
            has_nulls = vals.mask is not None and vals.null_count > 0
            nullable = kind in (Kind.VARIANCE, Kind.STD) or \
                (has_nulls and kind not in (Kind.COUNT_VALID, Kind.COUNT_ALL, Kind.M2))
            row.append(column(rtypes[i], res_bufs[i], res_masks[i], nulls[nk + i], nullable))
            i += 1
        out_res.append(row)
    return out_keys, out_res


def make_inputs(seed, n, groups):
    rng = np.random.default_rng(seed)
    a = HostColumn.from_numpy(rng.integers(-groups // 8, groups // 8, n).astype(np.int32), valid=rng.random(n) > 0.03)
    b = HostColumn.from_numpy(rng.integers(0, 4, n).astype(np.int16))
    v = HostColumn.from_numpy(rng.standard_normal(n), valid=rng.random(n) > 0.1)
    w = HostColumn.from_numpy(rng.integers(-1000, 1000, n).astype(np.int32))
    reqs = [(v, [Kind.SUM, Kind.COUNT_VALID, Kind.MEAN, Kind.MIN, Kind.MAX, Kind.VARIANCE]),
            (w, [Kind.SUM, Kind.COUNT_ALL, Kind.MAX])]
    return [a, b], reqs


def test_noalloc_matches_the_allocating_entry_point_twice_in_a_row():
    # two different inputs back to back: the second call must not see anything of the first
    from oracle import oracle
    for call, (seed, n, groups, policy) in enumerate(((1, 300_000, 4000, NullPolicy.EXCLUDE),
                                                      (2, 120_000, 600, NullPolicy.INCLUDE),
                                                      (1, 300_000, 4000, NullPolicy.EXCLUDE))):
        keys, reqs = make_inputs(seed, n, groups)
        got = run_noalloc(keys, reqs, policy, max_groups=8192, warmed_up=call > 0)
        exp = H.gpu_groupby(keys, reqs, policy)
        # the tolerance is relative to each group's Σ|x| / Σx² (see helpers.result_scales): both sides are
        # GPU sums with different summation orders
        orc = oracle.groupby(keys, reqs, policy)
        scales = H.reorder_scales(H.result_scales(keys, reqs, policy), orc[0], exp[0])
        H.assert_same_result(got, exp, reqs, scales=scales)
        # and against the CPU oracle directly, not only against the other GPU entry point
        H.assert_same_result(got, orc, reqs, scales=H.result_scales(keys, reqs, policy))


def test_noalloc_rejects_sizes_beyond_the_scratch_array():
    import cudf_b200 as cb
    keys, reqs = make_inputs(3, 1000, 50)
    with pytest.raises(ValueError, match="fixed scratch array holds"):
        run_noalloc(keys, reqs, NullPolicy.EXCLUDE, max_groups=5_000_000)
    with pytest.raises(cb.LogicError, match="more than max_groups groups"):
        run_noalloc(keys, reqs, NullPolicy.EXCLUDE, max_groups=8)
    with pytest.raises(cb.UnsupportedError):
        s = HostColumn.from_strings(["a", "b"] * 500)
        run_noalloc([s], reqs, NullPolicy.EXCLUDE, max_groups=64)
